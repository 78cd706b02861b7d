"""fp32 CPU restatement of the TinyTransformer forward and of generate_output.

Test infrastructure (see oracle/__init__.py).  Arithmetic is plain torch on the CPU in fp32, the
same library calls the reference makes (nn.functional.linear, scaled_dot_product_attention,
silu), so the results agree with the reference to fp32 round-off; tests/golden pins that.

Weights live in a dict with the reference's state_dict names.  ``init_state`` draws seeded
random-init weights with the reference's distributions (src/transformer.py:547-560: Xavier-uniform
linears, N(0, 0.02) embeddings, zero biases, unit norm weights) from its own generator stream.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from .arc_tokens import END, GridState, initial_state

SIZES = {  # src/transformer.py:728-745
    "tiny": dict(d_model=256, n_heads=4, n_layers=4, d_ff=704),
    "small": dict(d_model=768, n_heads=12, n_layers=4, d_ff=2048),
    "medium": dict(d_model=1024, n_heads=16, n_layers=8, d_ff=2752),
    "large": dict(d_model=1280, n_heads=20, n_layers=12, d_ff=3392),
}


@dataclass
class Config:  # field names and defaults of TransformerConfig (src/transformer.py:15-34)
    vocab_size: int = 14
    max_seq_len: int = 1863
    d_model: int = 128
    n_heads: int = 4
    d_ff: int = 320
    n_layers: int = 4
    dropout: float = 0.1
    num_examples: int = 1280
    max_x: int = 32
    max_y: int = 32
    max_z: int = 8
    rope_base: float = 10000.0
    norm_eps: float = 1e-5
    rope_type: str = "3d"
    norm_type: str = "rmsnorm"
    ffn_type: str = "swiglu"
    use_example_embedding: bool = True


def make_config(size: str, **kw) -> Config:
    return Config(**SIZES[size], **kw)


def init_state(cfg: Config, seed: int = 0, head_gain: float = 1.0, embed_gain: float = 1.0) -> dict:
    """Seeded random-init weights (fp32).  ``head_gain``/``embed_gain`` rescale lm_head and
    token_embed: the plain init generates one constant colour forever, a rescaled one gives
    varied tokens, which exercises NEWLINE / END / ragged-finish paths."""
    g = torch.Generator().manual_seed(seed)
    d, dff = cfg.d_model, cfg.d_ff

    def xavier(out_f, in_f):
        bound = math.sqrt(6.0 / (in_f + out_f))
        return (torch.rand(out_f, in_f, generator=g) * 2 - 1) * bound

    sd = {
        "token_embed.weight": torch.randn(cfg.vocab_size, d, generator=g) * 0.02 * embed_gain,
        "example_embed.weight": torch.randn(cfg.num_examples, d, generator=g) * 0.02,
    }
    for l in range(cfg.n_layers):
        p = f"blocks.{l}."
        sd[p + "ln1.weight"] = torch.ones(d)
        sd[p + "attn.qkv_proj.weight"] = xavier(3 * d, d)
        sd[p + "attn.out_proj.weight"] = xavier(d, d)
        sd[p + "ln2.weight"] = torch.ones(d)
        sd[p + "ffn.fc_gate.weight"] = xavier(dff, d)
        sd[p + "ffn.fc_gate.bias"] = torch.zeros(dff)
        sd[p + "ffn.fc_up.weight"] = xavier(dff, d)
        sd[p + "ffn.fc_up.bias"] = torch.zeros(dff)
        sd[p + "ffn.fc_down.weight"] = xavier(d, dff)
        sd[p + "ffn.fc_down.bias"] = torch.zeros(d)
    sd["ln_f.weight"] = torch.ones(d)
    sd["lm_head.weight"] = xavier(cfg.vocab_size, d) * head_gain
    return sd


def perturb_state(sd: dict, seed: int, scale: float = 0.05) -> dict:
    """Make biases and norm weights non-trivial (the init leaves them at 0 / 1), so that the bias
    and norm-weight code paths are actually exercised by parity tests."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for k, v in sd.items():
        if k.endswith(".bias") or ("ln" in k and k.endswith(".weight")):
            out[k] = v + torch.randn(v.shape, generator=g) * scale
        else:
            out[k] = v
    return out


def round_bf16(sd: dict) -> dict:
    """Parameters rounded to bf16 and held in fp32: the values the B200 kernels actually use."""
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in sd.items()}


def rope_tables(cfg: Config):  # src/transformer.py:87-126
    n_pairs = (cfg.d_model // cfg.n_heads) // 2
    px = py = n_pairs // 3
    pz = n_pairs - px - py

    def tab(n, pairs):
        dim = pairs * 2
        inv = 1.0 / (cfg.rope_base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        fr = torch.outer(torch.arange(n, dtype=torch.float32), inv)
        return fr.cos(), fr.sin()

    return tab(cfg.max_x, px), tab(cfg.max_y, py), tab(cfg.max_z, pz)


def _rotate_half(x):  # src/transformer.py:51-58
    return torch.stack((-x[..., 1::2], x[..., ::2]), dim=-1).flatten(-2)


def apply_rope(cfg: Config, tables, q, k, pos):  # src/transformer.py:132-187; q,k [B,S,H,64]
    (cx, sx), (cy, sy), (cz, sz) = tables
    xp = pos[..., 0].clamp(0, cfg.max_x - 1).long()
    yp = pos[..., 1].clamp(0, cfg.max_y - 1).long()
    zp = pos[..., 2].clamp(0, cfg.max_z - 1).long()
    cos = torch.cat([cx[xp].repeat_interleave(2, -1), cy[yp].repeat_interleave(2, -1),
                     cz[zp].repeat_interleave(2, -1)], -1).unsqueeze(2)
    sin = torch.cat([sx[xp].repeat_interleave(2, -1), sy[yp].repeat_interleave(2, -1),
                     sz[zp].repeat_interleave(2, -1)], -1).unsqueeze(2)
    return q * cos + _rotate_half(q) * sin, k * cos + _rotate_half(k) * sin


def rmsnorm(x, w, eps):  # src/transformer.py:45-48
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _sdpa_mask(mask_bool, dtype):  # src/inference.py:372-380
    return torch.where(mask_bool[:, None, None, :], 0.0, float("-inf")).to(dtype)


def _ffn(sd, p, x):  # src/transformer.py:446-451
    gate = F.silu(F.linear(x, sd[p + "ffn.fc_gate.weight"], sd[p + "ffn.fc_gate.bias"]))
    up = F.linear(x, sd[p + "ffn.fc_up.weight"], sd[p + "ffn.fc_up.bias"])
    return F.linear(gate * up, sd[p + "ffn.fc_down.weight"], sd[p + "ffn.fc_down.bias"])


def _embed(sd, cfg, ids, example_ids):
    x = sd["token_embed.weight"][ids]
    if cfg.use_example_embedding and example_ids is not None:
        x = x + sd["example_embed.weight"][example_ids].unsqueeze(1)
    return x


@torch.no_grad()
def forward(sd: dict, cfg: Config, ids, pos, example_ids=None, mask=None, is_causal=True, operand_dtype=None):
    """TinyTransformer.forward (src/transformer.py:562-599): logits [B, S, 14] in fp32.

    ``operand_dtype`` (torch.float16 / torch.bfloat16) is an error model, not the reference: every
    matmul and attention OPERAND that a 16-bit-activation pipeline stores in that format (both
    normalised streams, q, k, v, the attention output, the SwiGLU activations) is rounded to it and
    all arithmetic stays fp32.  It shows how far ANY such pipeline can be from the fp32 forward."""
    B, S = ids.shape
    H, hd = cfg.n_heads, cfg.d_model // cfg.n_heads
    tables = rope_tables(cfg)
    x = _embed(sd, cfg, ids, example_ids)
    amask = None if mask is None else _sdpa_mask(mask.bool(), x.dtype)

    def r(t):
        return t if operand_dtype is None else t.to(operand_dtype).to(torch.float32)

    for l in range(cfg.n_layers):
        p = f"blocks.{l}."
        h = r(rmsnorm(x, sd[p + "ln1.weight"], cfg.norm_eps))
        qkv = F.linear(h, sd[p + "attn.qkv_proj.weight"]).reshape(B, S, 3, H, hd)
        q, k, v = qkv.unbind(2)
        q, k = apply_rope(cfg, tables, q, k, pos)
        q, k, v = r(q), r(k), r(v)
        o = r(F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                             attn_mask=amask, is_causal=is_causal))
        x = x + F.linear(o.transpose(1, 2).reshape(B, S, -1), sd[p + "attn.out_proj.weight"])
        h2 = r(rmsnorm(x, sd[p + "ln2.weight"], cfg.norm_eps))
        if operand_dtype is None:
            x = x + _ffn(sd, p, h2)
        else:
            gate = F.silu(F.linear(h2, sd[p + "ffn.fc_gate.weight"], sd[p + "ffn.fc_gate.bias"]))
            up = F.linear(h2, sd[p + "ffn.fc_up.weight"], sd[p + "ffn.fc_up.bias"])
            x = x + F.linear(r(gate * up), sd[p + "ffn.fc_down.weight"], sd[p + "ffn.fc_down.bias"])
    return F.linear(rmsnorm(x, sd["ln_f.weight"], cfg.norm_eps), sd["lm_head.weight"])


def apply_constraints(logits, states, cons):
    """_apply_logit_constraints (src/inference.py:285-364) on logits [B, 14]; ``states`` are the
    per-row GridState objects (state after the last fed token).  ``cons`` is a dict with
    palette_mask [B,10] bool | None, target_shape [B,2] | None, palette_penalty, shape_penalty,
    disallow_tokens."""
    if cons is None:
        return logits
    logits = logits.clone()
    for tok in cons.get("disallow_tokens", (10, 12)):
        logits[:, tok] = float("-inf")
    pm = cons.get("palette_mask")
    if pm is not None:
        logits[:, :10] -= (~pm.bool()).to(logits.dtype) * cons.get("palette_penalty", 2.0)
    ts = cons.get("target_shape")
    if ts is not None:
        pen = cons.get("shape_penalty", 2.0)
        for b, st in enumerate(states):
            th, tw = int(ts[b, 0]), int(ts[b, 1])
            if th < 0 or tw < 0:
                continue
            if st.x >= tw:
                logits[b, :10] -= pen
            else:
                logits[b, 11] -= pen
            if st.y >= th:
                logits[b, :10] -= pen
                logits[b, 11] -= pen
    return logits


@dataclass
class GenResult:
    tokens: torch.Tensor                      # [B, S + n_generated] like generate_output
    logits: list = field(default_factory=list)  # per generated position: [B, 14]
    picked_from: list = field(default_factory=list)  # the logits the argmax saw (after constraints)


@torch.no_grad()
def generate(sd: dict, cfg: Config, ids, pos, example_ids=None, mask=None, max_new_tokens=900,
             stop_on_end=True, forced=None, keep_logits=False, constraints=None) -> GenResult:
    """generate_output, greedy branch (src/inference.py:487-628), with its helpers _prefill
    (383-424), _decode_step (427-459), StaticKVCache (51-96) and the grid-state tracker.

    ``forced`` [B, >= n] teacher-forces the fed tokens (logits are still those of the model).
    """
    B, S = ids.shape
    H, hd, L = cfg.n_heads, cfg.d_model // cfg.n_heads, cfg.n_layers
    if example_ids is None:
        example_ids = torch.zeros(B, dtype=torch.long)
    pmask = torch.ones(B, S, dtype=torch.bool) if mask is None else mask.bool()
    total = min(S + max_new_tokens, cfg.max_seq_len)
    max_new = total - S
    if max_new <= 0:
        return GenResult(ids)
    tables = rope_tables(cfg)
    cache = torch.zeros(L, 2, B, H, total, hd)
    lengths = pmask.long().sum(1)
    last_idx = (lengths - 1).clamp(min=0)
    ar = torch.arange(B)
    states = []
    for b in range(B):
        x0, y0, io = initial_state(int(ids[b, last_idx[b]]), pos[b, last_idx[b]].tolist(), bool(lengths[b] > 0))
        states.append(GridState(x0, y0, io))
    full_mask = torch.zeros(B, total, dtype=torch.bool)
    full_mask[:, :S] = pmask

    # prefill
    x = _embed(sd, cfg, ids, example_ids)
    amask = _sdpa_mask(pmask, x.dtype)
    for l in range(L):
        p = f"blocks.{l}."
        h = rmsnorm(x, sd[p + "ln1.weight"], cfg.norm_eps)
        q, k, v = F.linear(h, sd[p + "attn.qkv_proj.weight"]).reshape(B, S, 3, H, hd).unbind(2)
        q, k = apply_rope(cfg, tables, q, k, pos)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        cache[l, 0, :, :, :S] = k
        cache[l, 1, :, :, :S] = v
        o = F.scaled_dot_product_attention(q, cache[l, 0, :, :, :S], cache[l, 1, :, :, :S],
                                           attn_mask=amask, is_causal=True)
        x = x + F.linear(o.transpose(1, 2).reshape(B, S, -1), sd[p + "attn.out_proj.weight"])
        x = x + _ffn(sd, p, rmsnorm(x, sd[p + "ln2.weight"], cfg.norm_eps))
    logits = F.linear(rmsnorm(x[ar, last_idx], sd["ln_f.weight"], cfg.norm_eps), sd["lm_head.weight"])

    all_logits = [logits] if keep_logits else []
    used = apply_constraints(logits, states, constraints)
    used_logits = [used] if keep_logits else []
    nxt = used.argmax(-1)
    if forced is not None:
        nxt = forced[:, 0].long()
    out = [ids, nxt[:, None]]
    finished = torch.zeros(B, dtype=torch.bool)
    full_mask[:, S] = True
    if stop_on_end:
        finished |= nxt == END
    seq_len = S
    for step in range(1, max_new):
        if stop_on_end and forced is None and bool(finished.all()):
            break
        cur_pos = torch.tensor([states[b].update(int(nxt[b])) for b in range(B)], dtype=torch.long)[:, None, :]
        x = _embed(sd, cfg, nxt[:, None], example_ids)
        amask = _sdpa_mask(full_mask[:, :seq_len + 1], x.dtype)
        for l in range(L):
            p = f"blocks.{l}."
            h = rmsnorm(x, sd[p + "ln1.weight"], cfg.norm_eps)
            q, k, v = F.linear(h, sd[p + "attn.qkv_proj.weight"]).reshape(B, 1, 3, H, hd).unbind(2)
            q, k = apply_rope(cfg, tables, q, k, cur_pos)
            cache[l, 0, :, :, seq_len] = k[:, 0]
            cache[l, 1, :, :, seq_len] = v[:, 0]
            o = F.scaled_dot_product_attention(q.transpose(1, 2), cache[l, 0, :, :, :seq_len + 1],
                                               cache[l, 1, :, :, :seq_len + 1], attn_mask=amask, is_causal=False)
            x = x + F.linear(o.transpose(1, 2).reshape(B, 1, -1), sd[p + "attn.out_proj.weight"])
            x = x + _ffn(sd, p, rmsnorm(x, sd[p + "ln2.weight"], cfg.norm_eps))
        seq_len += 1
        logits = F.linear(rmsnorm(x, sd["ln_f.weight"], cfg.norm_eps), sd["lm_head.weight"])[:, 0]
        used = apply_constraints(logits, states, constraints)
        if keep_logits:
            all_logits.append(logits)
            used_logits.append(used)
        nxt = used.argmax(-1)
        if forced is not None:
            nxt = forced[:, step].long()
        if stop_on_end:
            finished |= nxt == END
        out.append(nxt[:, None])
        full_mask[:, S + step] = True
    return GenResult(torch.cat(out, 1), all_logits, used_logits)
