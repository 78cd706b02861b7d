"""Host wrapper over the C-ABI library: weight packing, sessions, packed prefill, graph decode.

torch is used only for device memory, streams and host<->device copies; every kernel that runs
is one of the library's own.  There is no CPU fallback: constructing an Engine without the
built library or without a B200 raises.
"""
from __future__ import annotations

import ctypes as C
import weakref
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from .data import END_TOKEN_ID, IO_SEP_TOKEN_ID, MAX_X, MAX_Y, NEWLINE_TOKEN_ID, START_TOKEN_ID

VOCAB = 14
HEAD_DIM = 64


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def sample_uniform(seed: int, stream: int, index: int) -> float:
    """The uniform number in [0, 1) that the token-picking kernel draws for generated token ``index``
    of the row whose random-stream id is ``stream`` (host mirror of the device's counter-based
    generator: splitmix64 of seed + golden * (stream + 1) + c * (index + 1), top 24 bits)."""
    m = (1 << 64) - 1
    z = (seed + 0x9E3779B97F4A7C15 * (stream + 1) + 0xD1B54A32D192ED03 * (index + 1)) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    z ^= z >> 31
    return (z >> 40) / 16777216.0


def rope_tables(head_dim: int, max_x: int, max_y: int, max_z: int, base: float) -> dict[str, torch.Tensor]:
    """cos/sin tables of RotaryEmbedding3D (src/transformer.py:87-126), fp32 on the CPU.

    The same torch ops in the same order as the reference, so the tables are bit-identical to
    the module's non-persistent buffers.
    """
    n_pairs = head_dim // 2
    px = n_pairs // 3
    py = n_pairs // 3
    pz = n_pairs - px - py

    def table(n_pos: int, pairs: int):
        dim = pairs * 2
        inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        freqs = torch.outer(torch.arange(n_pos, dtype=torch.float32), inv_freq)
        return freqs.cos(), freqs.sin()

    cx, sx = table(max_x, px)
    cy, sy = table(max_y, py)
    cz, sz = table(max_z, pz)
    return {"ROPE_COS_X": cx, "ROPE_SIN_X": sx, "ROPE_COS_Y": cy, "ROPE_SIN_Y": sy,
            "ROPE_COS_Z": cz, "ROPE_SIN_Z": sz}


_STATE_KEYS = {
    "TOKEN_EMBED": "token_embed.weight", "EXAMPLE_EMBED": "example_embed.weight",
    "LNF_W": "ln_f.weight", "LM_HEAD": "lm_head.weight",
}
_LAYER_KEYS = {
    "LN1_W": "ln1.weight", "QKV_W": "attn.qkv_proj.weight", "OUT_W": "attn.out_proj.weight",
    "LN2_W": "ln2.weight", "GATE_W": "ffn.fc_gate.weight", "GATE_B": "ffn.fc_gate.bias",
    "UP_W": "ffn.fc_up.weight", "UP_B": "ffn.fc_up.bias", "DOWN_W": "ffn.fc_down.weight",
    "DOWN_B": "ffn.fc_down.bias",
}


def _cfg_get(cfg, name, default=None):
    if isinstance(cfg, dict):
        return cfg.get(name, default)
    return getattr(cfg, name, default)


class Engine:
    """Packed bf16 weights of one TinyTransformer on one B200 (``arcb_engine``)."""

    def __init__(self, state_dict: dict, config, device="cuda:0", act_format: str = "f16",
                 gemm_path: str = "auto", attn_path: str = "auto"):
        self.lib = _lib.load()
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("the B200 engine needs a CUDA device; there is no CPU path")
        for name, want in (("rope_type", "3d"), ("norm_type", "rmsnorm"), ("ffn_type", "swiglu")):
            got = str(_cfg_get(config, name, want)).lower()
            if got != want:
                raise NotImplementedError(f"{name}={got!r} is not implemented (only {want!r})")
        self.d_model = int(_cfg_get(config, "d_model"))
        self.n_heads = int(_cfg_get(config, "n_heads"))
        self.n_layers = int(_cfg_get(config, "n_layers"))
        self.d_ff = int(_cfg_get(config, "d_ff"))
        self.vocab_size = int(_cfg_get(config, "vocab_size", VOCAB))
        self.max_seq_len = int(_cfg_get(config, "max_seq_len", 1863))
        self.num_examples = int(_cfg_get(config, "num_examples", 1280))
        self.use_example_embedding = bool(_cfg_get(config, "use_example_embedding", True))
        if self.vocab_size != VOCAB or self.d_model != self.n_heads * HEAD_DIM:
            raise NotImplementedError("only vocab_size 14 and head_dim 64 are implemented")
        self.act_format = {"f16": _lib.ACT_F16, "bf16": _lib.ACT_BF16}[act_format]
        cfg = _lib.Config(
            d_model=self.d_model, n_heads=self.n_heads, n_layers=self.n_layers, d_ff=self.d_ff,
            vocab_size=self.vocab_size, num_examples=self.num_examples,
            max_x=int(_cfg_get(config, "max_x", 32)), max_y=int(_cfg_get(config, "max_y", 32)),
            max_z=int(_cfg_get(config, "max_z", 8)),
            use_example_embedding=int(self.use_example_embedding), act_format=self.act_format,
            gemm_path={"auto": _lib.GEMM_AUTO, "simt": _lib.GEMM_SIMT, "tc": _lib.GEMM_TC}[gemm_path],
            attn_path={"auto": _lib.ATTN_AUTO, "stream": _lib.ATTN_STREAM}[attn_path],
            norm_eps=float(_cfg_get(config, "norm_eps", 1e-5)))
        self._handle = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.arcb_engine_create(C.byref(cfg), C.byref(self._handle)))
            tables = rope_tables(HEAD_DIM, cfg.max_x, cfg.max_y, cfg.max_z,
                                 float(_cfg_get(config, "rope_base", 10000.0)))
            for kind, t in tables.items():
                self._load(kind, 0, t)
            for kind, key in _STATE_KEYS.items():
                self._load(kind, 0, state_dict[key])
            for layer in range(self.n_layers):
                for kind, key in _LAYER_KEYS.items():
                    self._load(kind, layer, state_dict[f"blocks.{layer}.{key}"])
            torch.cuda.synchronize(self.device)

    @classmethod
    def from_module(cls, model, device="cuda:0", **kw) -> "Engine":
        """Build from a reference ``TinyTransformer`` (anything with ``.config`` + ``state_dict()``)."""
        return cls(model.state_dict(), model.config, device=device, **kw)

    def _load(self, kind: str, layer: int, t: torch.Tensor) -> None:
        src = t.detach().to(device=self.device, dtype=torch.float32).contiguous()
        _lib.check(self.lib.arcb_engine_load_tensor(self._handle, _lib.KIND[kind], layer, src.data_ptr(),
                                                    src.numel(), _stream_ptr(self.device)))
        torch.cuda.current_stream(self.device).synchronize()  # src may be a temporary

    def close(self) -> None:
        if getattr(self, "_handle", None) and self._handle.value:
            self.lib.arcb_engine_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def saturation_count(self, reset: bool = True) -> int:
        """Values clamped to the half range (or attention scores that overflowed it) since the last
        reset: a warning that the model's activations do not fit IEEE half (use act_format="bf16")."""
        n = C.c_int64(0)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.arcb_engine_saturation_count(self._handle, C.byref(n), int(bool(reset)),
                                                             _stream_ptr(self.device)))
        return int(n.value)

    # ------------------------------------------------------------------
    def kv_bytes_per_position(self) -> int:
        return self.n_layers * 2 * self.d_model * 2

    def new_session(self, n_seqs: int, t_max: int, max_new: int, max_prefill_tokens: int,
                    stop_on_end: bool = True, attn_splits: int = 0, forced: torch.Tensor | None = None,
                    want_step_logits: bool = False, out_tokens: torch.Tensor | None = None,
                    constraints: dict | None = None, temperature: float = 0.0, top_k: int = 0,
                    sample_seed: int = 0, sample_stream=None) -> "Session":
        return Session(self, n_seqs, t_max, max_new, max_prefill_tokens, stop_on_end, attn_splits,
                       forced, want_step_logits, out_tokens, constraints, temperature, top_k, sample_seed,
                       sample_stream)


_ENGINES: "weakref.WeakKeyDictionary" = weakref.WeakKeyDictionary()


def engine_for(model, device=None, **kw) -> Engine:
    """One cached Engine per live model object (weights are packed once)."""
    if device is None:
        device = next(model.parameters()).device
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("the B200 path needs the model (or the device argument) on a CUDA device")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = (str(device), tuple(sorted(kw.items())))
    per_model = _ENGINES.setdefault(model, {})
    if key not in per_model:
        per_model[key] = Engine.from_module(model, device=device, **kw)
    return per_model[key]


def cache_row_pitch(t_max: int) -> int:
    """Rows reserved per (sequence, head) in the KV cache for a requested capacity of ``t_max`` rows:
    the smallest value >= t_max that is 16 modulo 32, i.e. a distance between two streams that is an
    odd multiple of 2 KB.  Decode attention reads thousands of such streams at once; when their
    distance is a multiple of 64 KB (1536 rows, 2048 rows) the streams fall on the same memory channels
    in step and the measured read bandwidth is 2.5-3 % lower (7.05-7.09 TB/s against 6.84-6.90 TB/s at
    1024 sequences x 20 heads x 717 cached rows, 1552 against 1536 rows)."""
    t = int(t_max)
    return t + ((16 - t) % 32)


class Session:
    """A static KV cache, the greedy-loop state and the decode graph for ``n_seqs`` sequences.
    ``t_max`` is the capacity asked for; ``self.t_max`` is the row pitch the cache is laid out with
    (``cache_row_pitch``), which is what the library is given as its ``t_max``."""

    def __init__(self, eng: Engine, n_seqs, t_max, max_new, max_prefill_tokens, stop_on_end,
                 attn_splits, forced, want_step_logits, out_tokens=None, constraints=None,
                 temperature=0.0, top_k=0, sample_seed=0, sample_stream=None):
        self.eng = eng
        self.n_seqs, self.t_max, self.max_new = int(n_seqs), cache_row_pitch(t_max), int(max_new)
        self.t_requested = int(t_max)
        self.max_prefill_tokens = int(max_prefill_tokens)
        dev = eng.device
        lib = eng.lib
        kv_bytes = lib.arcb_kv_cache_bytes(eng._handle, self.n_seqs, self.t_max)
        ws_bytes = lib.arcb_session_workspace_bytes(eng._handle, self.n_seqs, self.max_prefill_tokens,
                                                    int(attn_splits))
        if kv_bytes <= 0 or ws_bytes <= 0:
            raise ValueError("bad session sizes")
        # torch owns the memory; the library only borrows the pointers
        self.kv_cache = torch.empty(kv_bytes, dtype=torch.uint8, device=dev)
        self.workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        if out_tokens is None:
            out_tokens = torch.full((self.n_seqs, self.max_new), END_TOKEN_ID, dtype=torch.int32, device=dev)
        elif (out_tokens.dtype != torch.int32 or tuple(out_tokens.shape) != (self.n_seqs, self.max_new)
              or not out_tokens.is_contiguous() or out_tokens.device != dev):
            raise ValueError("out_tokens must be a contiguous int32 [n_seqs, max_new] tensor on the engine's device")
        self.out_tokens = out_tokens  # may be a slice of a caller-owned (e.g. all-gather) buffer
        self.forced = None
        if forced is not None:
            self.forced = forced.to(device=dev, dtype=torch.int32).contiguous()
            assert self.forced.shape == (self.n_seqs, self.max_new)
        self.step_logits = (torch.zeros((self.n_seqs, self.max_new, VOCAB), dtype=torch.float32, device=dev)
                            if want_step_logits else None)
        # soft decoding constraints: dict(palette_mask=[B,10] bool|None, target_shape=[B,2] int|None,
        # palette_penalty, shape_penalty, disallow_tokens)
        self.palette_mask = self.target_shape = None
        pal_pen = shp_pen = 0.0
        disallow = 0
        if constraints is not None:
            pm, ts = constraints.get("palette_mask"), constraints.get("target_shape")
            if pm is not None:
                self.palette_mask = torch.as_tensor(pm).to(device=dev, dtype=torch.uint8).contiguous()
                assert tuple(self.palette_mask.shape) == (self.n_seqs, 10)
            if ts is not None:
                self.target_shape = torch.as_tensor(ts).to(device=dev, dtype=torch.int32).contiguous()
                assert tuple(self.target_shape.shape) == (self.n_seqs, 2)
            pal_pen = float(constraints.get("palette_penalty", 2.0))
            shp_pen = float(constraints.get("shape_penalty", 2.0))
            for t in constraints.get("disallow_tokens", ()):
                disallow |= 1 << int(t)
        # random-stream id of each row when sampling (default: the row index); a job split over
        # several sessions / ranks passes job-wide ids so that no two of its sequences share a stream
        self.sample_stream = None
        if sample_stream is not None:
            self.sample_stream = torch.as_tensor(np.asarray(sample_stream, dtype=np.int64) & 0x7FFFFFFF).to(
                device=dev, dtype=torch.int32).contiguous()
            assert tuple(self.sample_stream.shape) == (self.n_seqs,)
        desc = _lib.SessionDesc(
            n_seqs=self.n_seqs, t_max=self.t_max, max_new=self.max_new,
            max_prefill_tokens=self.max_prefill_tokens, attn_splits=int(attn_splits),
            stop_on_end=(2 if stop_on_end == 2 else int(bool(stop_on_end))),
            d_kv_cache=self.kv_cache.data_ptr(), kv_cache_bytes=kv_bytes,
            d_workspace=self.workspace.data_ptr(), workspace_bytes=ws_bytes,
            d_out_tokens=self.out_tokens.data_ptr(), d_forced=_ptr(self.forced),
            d_step_logits=_ptr(self.step_logits),
            d_palette_mask=_ptr(self.palette_mask), d_target_shape=_ptr(self.target_shape),
            palette_penalty=pal_pen, shape_penalty=shp_pen, disallow_token_mask=disallow,
            temperature=float(temperature), top_k=int(top_k or 0), sample_seed=int(sample_seed) & (2 ** 64 - 1),
            d_sample_stream=_ptr(self.sample_stream))
        self._handle = C.c_void_p()
        with torch.cuda.device(dev):
            _lib.check(lib.arcb_session_create(eng._handle, C.byref(desc), C.byref(self._handle)))

    def close(self) -> None:
        """Destroy the library session and give the cache and workspace back to torch's allocator
        (work already queued on the stream still completes first: the allocator is stream-ordered)."""
        if getattr(self, "_handle", None) and self._handle.value:
            self.eng.lib.arcb_session_destroy(self._handle)
            self._handle = C.c_void_p()
        self.kv_cache = None
        self.workspace = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def prefill(self, plan: "PrefillPlan", example_ids: torch.Tensor | None,
                logits_all: torch.Tensor | None = None, first_logits: torch.Tensor | None = None) -> None:
        """Run one packed-prompt forward (arcb_prefill). ``plan`` tensors are on the device."""
        a = _lib.PrefillArgs(
            n_tokens=plan.n_tokens, d_token_ids=_ptr(plan.token_ids), d_pos_xyz=_ptr(plan.pos_xyz),
            d_seq=_ptr(plan.seq), d_kv_slot=_ptr(plan.kv_slot), d_kv_count=_ptr(plan.kv_count),
            d_example_ids=_ptr(example_ids),
            n_qblocks=plan.n_qblocks, d_qblock_row0=_ptr(plan.qblock_row0), d_qblock_rows=_ptr(plan.qblock_rows),
            d_qblock_kv0=_ptr(plan.qblock_kv0), d_kv_row=_ptr(plan.kv_row), n_kv_rows=plan.n_kv_rows,
            kv_row_identity=int(bool(plan.kv_row_identity)),
            d_logits_all=_ptr(logits_all),
            n_first=plan.n_first, d_first_row=_ptr(plan.first_row), d_first_seq=_ptr(plan.first_seq),
            d_prompt_len=_ptr(plan.prompt_len), d_grid_x=_ptr(plan.grid_x), d_grid_y=_ptr(plan.grid_y),
            d_grid_in_output=_ptr(plan.grid_in_output), d_first_logits=_ptr(first_logits))
        with torch.cuda.device(self.eng.device):
            _lib.check(self.eng.lib.arcb_prefill(self._handle, C.byref(a), _stream_ptr(self.eng.device)))

    def decode(self, n_steps: int) -> None:
        with torch.cuda.device(self.eng.device):
            _lib.check(self.eng.lib.arcb_decode(self._handle, int(n_steps), _stream_ptr(self.eng.device)))

    def attention_probe_ms(self) -> float:
        """Device time of the layer-0 decode-attention launch of the most recent decode step."""
        ms = C.c_float(0)
        _lib.check(self.eng.lib.arcb_session_attention_probe(self._handle, C.byref(ms)))
        return float(ms.value)

    def poll(self) -> int:
        """Synchronise and return the number of rows that have emitted END; raises on a device error."""
        nf, err = C.c_int32(0), C.c_int32(0)
        with torch.cuda.device(self.eng.device):
            _lib.check(self.eng.lib.arcb_session_poll(self._handle, C.byref(nf), C.byref(err),
                                                      _stream_ptr(self.eng.device)))
        return int(nf.value)


# ---------------------------------------------------------------------------
# host-side planning of a packed prefill
# ---------------------------------------------------------------------------
@dataclass
class PrefillPlan:
    n_tokens: int
    token_ids: torch.Tensor
    pos_xyz: torch.Tensor
    seq: torch.Tensor
    kv_slot: torch.Tensor
    kv_count: torch.Tensor
    n_qblocks: int
    qblock_row0: torch.Tensor | None
    qblock_rows: torch.Tensor | None
    qblock_kv0: torch.Tensor | None = None   # first K/V scratch row of each block's sequence
    kv_row: torch.Tensor | None = None       # K/V scratch row of each token (-1: query-only)
    n_kv_rows: int = 0
    n_first: int = 0
    first_row: torch.Tensor | None = None
    first_seq: torch.Tensor | None = None
    prompt_len: torch.Tensor | None = None
    grid_x: torch.Tensor | None = None
    grid_y: torch.Tensor | None = None
    grid_in_output: torch.Tensor | None = None
    kv_row_identity: bool = False   # kv_row[i] == i for i < n_kv_rows and < 0 after

    def to(self, device) -> "PrefillPlan":
        def mv(t):
            return None if t is None else t.to(device, non_blocking=True)
        return PrefillPlan(self.n_tokens, mv(self.token_ids), mv(self.pos_xyz), mv(self.seq), mv(self.kv_slot),
                           mv(self.kv_count), self.n_qblocks, mv(self.qblock_row0), mv(self.qblock_rows),
                           mv(self.qblock_kv0), mv(self.kv_row), self.n_kv_rows,
                           self.n_first, mv(self.first_row), mv(self.first_seq), mv(self.prompt_len),
                           mv(self.grid_x), mv(self.grid_y), mv(self.grid_in_output), self.kv_row_identity)

    def h2d_bytes(self) -> int:
        n = 0
        for t in (self.token_ids, self.pos_xyz, self.seq, self.kv_slot, self.kv_count, self.qblock_row0,
                  self.qblock_rows, self.qblock_kv0, self.kv_row, self.first_row, self.first_seq, self.prompt_len, self.grid_x, self.grid_y,
                  self.grid_in_output):
            if t is not None:
                n += t.numel() * t.element_size()
        return n


def initial_grid_state(last_tok: np.ndarray, last_pos: np.ndarray, has_tokens: np.ndarray):
    """Grid state after the prompt (``_derive_initial_state_from_prompt``, src/inference.py:171-221).

    ``last_tok``/``last_pos`` are the token and position at index ``clamp(len-1, 0)`` of each row,
    read literally from the padded arrays as the reference does.
    """
    x, y, z = last_pos[:, 0].copy(), last_pos[:, 1].copy(), last_pos[:, 2]
    in_out = z >= 3
    is_start, is_sep = last_tok == START_TOKEN_ID, last_tok == IO_SEP_TOKEN_ID
    is_nl, is_color = last_tok == NEWLINE_TOKEN_ID, last_tok < 10
    in_out = np.where(is_start, False, in_out)
    in_out = np.where(is_sep, True, in_out)
    x = np.where(is_start | is_sep, 0, x)
    y = np.where(is_start | is_sep, 0, y)
    x = np.where(is_nl, 0, x)
    y = np.where(is_nl, np.minimum(y + 1, MAX_Y), y)
    x = np.where(is_color, np.minimum(x + 1, MAX_X), x)
    x = np.clip(x, 0, MAX_X)
    y = np.clip(y, 0, MAX_Y)
    x = np.where(has_tokens, x, 0)
    y = np.where(has_tokens, y, 0)
    in_out = np.where(has_tokens, in_out, True)
    return x.astype(np.int32), y.astype(np.int32), in_out.astype(np.int32)


def _qblocks(seq_of_row: np.ndarray, block: int = 256):
    """Split consecutive rows of the same sequence into blocks of at most ``block`` rows."""
    n = len(seq_of_row)
    if n == 0:
        return np.zeros(0, np.int32), np.zeros(0, np.int32)
    change = np.flatnonzero(np.diff(seq_of_row)) + 1
    starts = np.concatenate([[0], change])
    ends = np.concatenate([change, [n]])
    row0, rows = [], []
    for s, e in zip(starts.tolist(), ends.tolist()):
        for r in range(s, e, block):
            row0.append(r)
            rows.append(min(block, e - r))
    return np.asarray(row0, np.int32), np.asarray(rows, np.int32)


def plan_prefill(ids: np.ndarray, pos: np.ndarray, mask: np.ndarray, rows: np.ndarray,
                 is_causal: bool = True, all_positions: bool = False, with_first: bool = True) -> PrefillPlan:
    """Pack the sequences ``rows`` of a padded batch into one prefill call (host tensors).

    Valid positions become rows that store K/V at their compacted index and attend to the valid
    keys at or before them (causal AND key-padding, src/inference.py:409).  With
    ``all_positions`` padded positions are added as query-only rows (TinyTransformer.forward
    returns logits for them too).  The first generated token is read at padded index
    ``clamp(len-1, 0)`` exactly as ``_prefill`` does (src/inference.py:420-423): when that index
    is a padded position (left-padded rows), a query-only row is appended for it.
    """
    ids = ids[rows]
    pos = pos[rows]
    mask = mask[rows].astype(bool)
    n, S = ids.shape
    csum = np.cumsum(mask, axis=1)                       # valid keys at or before each index
    lens = csum[:, -1] if S > 0 else np.zeros(n, np.int64)
    sel = np.ones_like(mask) if all_positions else mask
    bi, si = np.nonzero(sel)                              # row-major: grouped by sequence, in order
    valid = mask[bi, si]
    tok = ids[bi, si].astype(np.int32)
    pxyz = pos[bi, si].astype(np.int32)
    seq = rows[bi].astype(np.int32)
    slot = np.where(valid, csum[bi, si] - 1, -1).astype(np.int32)
    if is_causal:
        cnt = csum[bi, si].astype(np.int32)
    else:
        cnt = lens[bi].astype(np.int32)
    plan_first = {}
    n_first = 0
    if with_first:
        last_idx = np.clip(lens - 1, 0, None)
        ar = np.arange(n)
        last_valid = mask[ar, last_idx]
        row_start = np.concatenate([[0], np.cumsum(sel.sum(axis=1))[:-1]])
        if all_positions:
            first_row = row_start + last_idx
        else:
            first_row = row_start + csum[ar, last_idx] - 1
        extra = np.flatnonzero(~last_valid)
        if len(extra) and not all_positions:
            # query-only rows for padded "last" positions, appended after the packed prompts
            base = len(tok)
            tok = np.concatenate([tok, ids[extra, last_idx[extra]].astype(np.int32)])
            pxyz = np.concatenate([pxyz, pos[extra, last_idx[extra]].astype(np.int32)])
            seq = np.concatenate([seq, rows[extra].astype(np.int32)])
            slot = np.concatenate([slot, np.full(len(extra), -1, np.int32)])
            cnt_extra = csum[extra, last_idx[extra]] if is_causal else lens[extra]
            cnt = np.concatenate([cnt, cnt_extra.astype(np.int32)])
            first_row = first_row.copy()
            first_row[extra] = base + np.arange(len(extra))
        gx, gy, gin = initial_grid_state(ids[ar, last_idx], pos[ar, last_idx], lens > 0)
        n_first = n
        plan_first = dict(
            first_row=torch.from_numpy(first_row.astype(np.int32)),
            first_seq=torch.from_numpy(rows.astype(np.int32)),
            prompt_len=torch.from_numpy(lens.astype(np.int32)),
            grid_x=torch.from_numpy(gx), grid_y=torch.from_numpy(gy), grid_in_output=torch.from_numpy(gin))
    qb0, qbn = _qblocks(seq)
    # K/V scratch of the call: the valid keys of sequence i occupy rows [kv_base[i], kv_base[i] + len_i)
    kv_base = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int64)
    local = np.searchsorted(rows, seq)  # index of each token's sequence within this call (rows is sorted)
    kv_row = np.where(slot >= 0, kv_base[local] + slot, -1).astype(np.int32)
    qb_kv0 = kv_base[local[qb0]].astype(np.int32) if len(qb0) else np.zeros(0, np.int32)
    if len(qb0):
        # most expensive query blocks first (cost = keys visible to the block's last row): the
        # attention kernel's CTAs are dispatched in this order, so its tail is made of cheap blocks
        order = np.argsort(-cnt[qb0 + qbn - 1].astype(np.int64), kind="stable")
        qb0, qbn, qb_kv0 = qb0[order], qbn[order], qb_kv0[order]
    n_kv = int(lens.sum())
    identity = bool(np.array_equal(kv_row[:n_kv], np.arange(n_kv, dtype=np.int32)) and (kv_row[n_kv:] < 0).all())
    return PrefillPlan(
        n_tokens=len(tok), token_ids=torch.from_numpy(tok), pos_xyz=torch.from_numpy(np.ascontiguousarray(pxyz)),
        seq=torch.from_numpy(seq), kv_slot=torch.from_numpy(slot), kv_count=torch.from_numpy(cnt),
        n_qblocks=len(qb0), qblock_row0=torch.from_numpy(qb0), qblock_rows=torch.from_numpy(qbn),
        qblock_kv0=torch.from_numpy(qb_kv0), kv_row=torch.from_numpy(kv_row), n_kv_rows=int(lens.sum()),
        n_first=n_first, kv_row_identity=identity, **plan_first)


def chunk_rows(lens: np.ndarray, max_tokens: int) -> list[np.ndarray]:
    """Greedy split of sequence indices into chunks whose packed token count fits ``max_tokens``."""
    chunks, cur, tot = [], [], 0
    for i, n in enumerate(lens.tolist()):
        n = max(int(n), 1) + 1  # +1: room for a possible query-only row
        if cur and tot + n > max_tokens:
            chunks.append(np.asarray(cur, np.int64))
            cur, tot = [], 0
        cur.append(i)
        tot += n
    if cur:
        chunks.append(np.asarray(cur, np.int64))
    return chunks
