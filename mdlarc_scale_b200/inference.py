"""Drop-in for the reference's generation API (``src/inference.py``) on the B200 engine.

``generate_output`` and ``predict_with_augmentations`` keep the reference's signatures, argument
meaning and error behaviour: greedy decoding, temperature / top-k sampling and the soft palette /
shape constraints all run on the device (sampling uses a counter-based random stream seeded from
torch's default generator; it cannot reproduce ``torch.multinomial`` draw for draw).

Differences from the reference that are part of the design:
  * prompts are packed (no padded positions are computed) and the KV cache is compacted, which
    is exact because attention is permutation-invariant over keys and positions enter only
    through the (x, y, z) RoPE;
  * by default a row that has emitted END is frozen and keeps emitting END, whereas the reference
    keeps decoding such rows until every row of its batch has finished (src/inference.py:593-626);
    rows agree through their first END.  The reference reads a candidate grid after the LAST IO_SEP of
    the whole row (src/inference.py:906-915), so a finished row that goes on to emit another IO_SEP
    changes its candidate there and not here.  ``freeze_finished=False`` (``generate_output``,
    ``predict_with_augmentations``) reproduces the reference's behaviour token for token.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .data import (DIHEDRAL_TRANSFORMS, END_TOKEN_ID, IO_SEP_TOKEN_ID, apply_color_perm_grid, as_rect_array,
                   compute_positions_3d, decode_output_grid, dihedral_np, encode_example, encode_example_np,
                   generate_color_permutations)
from .engine import Engine, Session, chunk_rows, engine_for, plan_prefill

DEFAULT_PREFILL_TOKENS = 65536  # packed prompt tokens per prefill call (bounds the workspace)
POLL_EVERY = 32                 # decode steps between two host checks of the finished counter


@dataclass(frozen=True)
class DecodingConstraints:
    """Soft decoding constraints with the reference's fields (src/inference.py:36-43): applied on the
    device, inside the kernel that picks the next token."""
    palette_mask: torch.Tensor | None = None   # [batch, 10] bool, True = colour allowed
    target_shape: torch.Tensor | None = None   # [batch, 2] (h, w), negative = no constraint
    palette_penalty: float = 2.0
    shape_penalty: float = 2.0
    disallow_tokens: tuple = (10, 12)          # START, IO_SEP


def _constraints_dict(constraints, batch: int) -> dict | None:
    """Host arrays for the session; batch broadcasting as in _apply_logit_constraints
    (src/inference.py:298-347): [1, n] rows are expanded, any other mismatch drops that constraint."""
    if constraints is None:
        return None

    def fit(t, width, dtype):
        if t is None:
            return None
        arr = np.asarray(t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else t)
        arr = arr.reshape(-1, width)
        if arr.shape[0] == 1 and batch != 1:
            arr = np.repeat(arr, batch, axis=0)
        return arr.astype(dtype) if arr.shape[0] == batch else None

    return dict(palette_mask=fit(constraints.palette_mask, 10, np.uint8),
                target_shape=fit(constraints.target_shape, 2, np.int32),
                palette_penalty=float(constraints.palette_penalty), shape_penalty=float(constraints.shape_penalty),
                disallow_tokens=tuple(int(t) for t in constraints.disallow_tokens))


@dataclass
class GenerationTrace:
    """Extra outputs of ``generate_tokens`` used by the parity harness and the benchmark."""
    tokens: torch.Tensor                 # int32 [B, n_generated] on the device
    first_logits: torch.Tensor | None    # fp32 [B, 14]
    step_logits: torch.Tensor | None     # fp32 [B, max_new, 14]
    prefill_tokens: int = 0
    decode_steps: int = 0
    h2d_bytes: int = 0


def _resolve_engine(model, device) -> Engine:
    """Engine for ``model``: on ``device`` if it is a CUDA device, else where the model lives,
    else the current CUDA device.  Raises when no CUDA device exists (there is no CPU path)."""
    if isinstance(model, Engine):
        return model
    if device is not None and torch.device(device).type == "cuda":
        return engine_for(model, device=device)
    p = next(model.parameters(), None)
    if p is not None and p.device.type == "cuda":
        return engine_for(model, device=p.device)
    if not torch.cuda.is_available():
        raise RuntimeError("mdlarc_scale_b200 needs a B200 GPU: no CUDA device is available and "
                           "there is no CPU fallback")
    return engine_for(model, device=torch.device("cuda", torch.cuda.current_device()))


def generate_tokens(engine: Engine, ids: np.ndarray, pos: np.ndarray, mask: np.ndarray,
                    example_ids: np.ndarray | None, max_new: int, stop_on_end: bool = True,
                    forced: np.ndarray | None = None, want_logits: bool = False,
                    max_prefill_tokens: int = DEFAULT_PREFILL_TOKENS, attn_splits: int = 0,
                    session: Session | None = None, pinned: bool = False,
                    constraints: dict | None = None, temperature: float = 0.0, top_k: int | None = None,
                    sample_seed: int = 0, freeze_finished: bool = True) -> GenerationTrace:
    """Prefill + greedy decode of a padded batch given as host arrays; returns device tokens.

    ``ids`` int [B, S], ``pos`` int [B, S, 3], ``mask`` bool [B, S] (True = real token).  At most
    ``max_new`` tokens are generated per row.  ``forced`` ([B, max_new]) teacher-forces the fed
    tokens while logits and argmax are still produced for every step.  With ``stop_on_end`` a row
    that has emitted END is frozen (it emits END from then on and its attention is skipped) unless
    ``freeze_finished`` is False, in which case it keeps decoding until every row has emitted END,
    which is what the reference does.
    """
    dev = engine.device
    B, S = ids.shape
    lens = mask.sum(axis=1)
    t_max = int(lens.max()) + int(max_new)
    cap = int(min(max_prefill_tokens, int(lens.sum()) + 2 * B))
    cap = max(cap, int(lens.max()) + 2, B)
    if session is None:
        session = engine.new_session(
            B, t_max, max_new, cap, stop_on_end=(2 if stop_on_end and not freeze_finished else stop_on_end),
            attn_splits=attn_splits,
            forced=None if forced is None else torch.from_numpy(np.ascontiguousarray(forced, dtype=np.int32)),
            want_step_logits=want_logits, constraints=constraints, temperature=temperature,
            top_k=top_k or 0, sample_seed=sample_seed)
    ex_dev = None
    h2d = 0
    if example_ids is not None and engine.use_example_embedding:
        ex_host = torch.from_numpy(np.ascontiguousarray(example_ids, dtype=np.int32))
        if pinned:
            ex_host = ex_host.pin_memory()
        ex_dev = ex_host.to(dev, non_blocking=True)
        h2d += ex_host.numel() * 4
    first_logits = torch.zeros((B, 14), dtype=torch.float32, device=dev) if want_logits else None
    n_prefill = 0
    for rows in chunk_rows(lens, session.max_prefill_tokens):
        plan = plan_prefill(ids, pos, mask, rows)
        h2d += plan.h2d_bytes()
        n_prefill += plan.n_tokens
        fl = None
        if first_logits is not None:
            fl = torch.zeros((len(rows), 14), dtype=torch.float32, device=dev)
        session.prefill(plan.to(dev), ex_dev, first_logits=fl)
        if fl is not None:
            first_logits[torch.from_numpy(rows).to(dev)] = fl
    steps_total = max_new - 1
    done = 0
    while done < steps_total:
        n = min(POLL_EVERY, steps_total - done) if stop_on_end and forced is None else steps_total - done
        session.decode(n)
        done += n
        if stop_on_end and forced is None and done < steps_total and session.poll() >= B:
            break
    session.poll()  # synchronise and surface any device-side error word
    n_gen = done + 1
    toks = session.out_tokens[:, :n_gen]
    if stop_on_end and forced is None:
        # the reference stops as soon as every row has emitted END (src/inference.py:594)
        is_end = toks == END_TOKEN_ID
        if bool(is_end.any(dim=1).all()):
            first_end = is_end.to(torch.int32).argmax(dim=1)
            n_gen = int(first_end.max().item()) + 1
            toks = toks[:, :n_gen]
    return GenerationTrace(tokens=toks, first_logits=first_logits, step_logits=session.step_logits,
                           prefill_tokens=n_prefill, decode_steps=done, h2d_bytes=h2d)


def generate_output(model, input_ids: torch.Tensor, positions_3d: torch.Tensor,
                    example_ids: torch.Tensor | None = None, attention_mask: torch.Tensor | None = None,
                    max_new_tokens: int = 900, temperature: float = 0.0, top_k: int | None = None,
                    stop_on_end: bool = True, use_compile: bool = False, constraints=None, *,
                    freeze_finished: bool = True) -> torch.Tensor:
    """Greedy generation with a static KV cache; same contract as ``src/inference.py:487-628``.

    ``model`` is a reference ``TinyTransformer`` (its weights are packed once and cached) or an
    ``Engine``.  Returns ``[batch, seq_len + n_generated]`` int64 on ``input_ids.device``.
    ``use_compile`` is accepted and ignored: the decode step always runs as a CUDA graph.
    ``temperature > 0`` samples (optionally from the ``top_k`` largest logits) instead of argmax.
    ``freeze_finished=False`` keeps decoding rows that have already emitted END until all rows have (the
    reference's exact behaviour; the default freezes them, which agrees through each row's first END).
    """
    batch, prompt_len = input_ids.shape
    if attention_mask is not None and tuple(attention_mask.shape) != (batch, prompt_len):
        raise ValueError("attention_mask must have shape [batch, seq_len]")
    if isinstance(model, Engine):
        engine = model
    else:
        model.eval()
        engine = _resolve_engine(model, input_ids.device)
    max_total = min(prompt_len + max_new_tokens, engine.max_seq_len)
    max_new = max_total - prompt_len
    if max_new <= 0:
        return input_ids
    ids = input_ids.detach().cpu().numpy()
    pos = positions_3d.detach().cpu().numpy()
    mask = (np.ones((batch, prompt_len), dtype=bool) if attention_mask is None
            else attention_mask.detach().to(torch.bool).cpu().numpy())
    ex = (np.zeros(batch, dtype=np.int64) if example_ids is None else example_ids.detach().cpu().numpy())
    seed = 0
    if temperature > 0:
        # one draw from torch's default generator per call, so torch.manual_seed makes sampling
        # reproducible as it does for the reference (whose torch.multinomial stream cannot be matched)
        seed = int(torch.randint(0, 2 ** 62, (1,)).item())
    trace = generate_tokens(engine, ids, pos, mask, ex, max_new, stop_on_end=stop_on_end,
                            constraints=_constraints_dict(constraints, batch), temperature=float(temperature),
                            top_k=top_k, sample_seed=seed, freeze_finished=freeze_finished)
    gen = trace.tokens.to(device=input_ids.device, dtype=input_ids.dtype)
    return torch.cat([input_ids, gen], dim=1)


def _grid_after_last_sep(tokens: list[int]):
    seps = [i for i, t in enumerate(tokens) if t == IO_SEP_TOKEN_ID]
    return decode_output_grid(tokens[seps[-1]:]) if seps else None


def predict_grid(model, input_grids, output_grids, test_input, device, example_id: int = 0,
                 max_output_tokens: int = 900, temperature: float = 0.0, top_k: int | None = None,
                 use_compile: bool = False, constraints: "DecodingConstraints | None" = None):
    """Output grid predicted for ``test_input`` given the training pairs, or None when nothing
    decodable follows the last IO_SEP (``src/inference.py:631-694``): one unpadded prompt through
    ``generate_output`` with END stopping."""
    toks: list[int] = []
    for inp, out in zip(input_grids, output_grids, strict=True):
        toks += encode_example(inp, out)
    toks += encode_example(test_input, None)
    device = torch.device(device)
    ids = torch.tensor([toks], dtype=torch.long, device=device)
    pos = torch.from_numpy(compute_positions_3d(toks)[None]).to(device)
    out = generate_output(model, ids, pos, torch.tensor([example_id], dtype=torch.long, device=device),
                          max_new_tokens=max_output_tokens, temperature=temperature, top_k=top_k,
                          stop_on_end=True, constraints=constraints)
    return _grid_after_last_sep(out[0].cpu().tolist())


def build_augmented_prompts(task: dict, test_idx: int, use_train_examples: bool = True,
                            num_color_perms: int = 8, num_samples: int = 1):
    """All (dihedral x colour-permutation x sample) prompts of one test input, in the reference's
    candidate order (src/inference.py:794-827): dihedral-major, then permutation, then sample.

    Returns ``(prompts, positions, aug_info)`` with ``aug_info[i] = (dihedral_idx, perm_tuple|None)``.
    """
    train_pairs = task["train"] if use_train_examples else []
    test_input = task["test"][test_idx]["input"]
    perms = generate_color_permutations(num_color_perms, seed=42)
    prompts, positions, info = [], [], []
    # vectorised path for well-formed (rectangular, colours 0-9) grids: same tokens and positions
    arrs = [(as_rect_array(p["input"]), as_rect_array(p["output"])) for p in train_pairs]
    t_arr = as_rect_array(test_input)
    if t_arr is not None and all(a is not None and b is not None for a, b in arrs) and \
            all(int(g.min()) >= 0 and int(g.max()) <= 9 for pair in arrs + [(t_arr, t_arr)] for g in pair):
        for d_idx in range(8):
            d_in = [dihedral_np(a, d_idx) for a, _ in arrs]
            d_out = [dihedral_np(b, d_idx) for _, b in arrs]
            d_tst = dihedral_np(t_arr, d_idx)
            for p_idx in range(num_color_perms):
                lut = perms[p_idx]
                tag = tuple(int(v) for v in lut) if p_idx > 0 else None
                parts = [encode_example_np(lut[gi], lut[go]) for gi, go in zip(d_in, d_out)]
                parts.append(encode_example_np(lut[d_tst], None))
                toks = np.concatenate([t for t, _ in parts])
                pos = np.concatenate([q for _, q in parts])
                for _ in range(max(1, num_samples)):
                    prompts.append(toks)
                    positions.append(pos)
                    info.append((d_idx, tag))
        return prompts, positions, info
    for d_idx, fn in enumerate(DIHEDRAL_TRANSFORMS):
        ins = [fn(p["input"]) for p in train_pairs]
        outs = [fn(p["output"]) for p in train_pairs]
        tst = fn(test_input)
        for p_idx in range(num_color_perms):
            perm = perms[p_idx]
            if p_idx > 0:
                p_ins = [apply_color_perm_grid(g, perm) for g in ins]
                p_outs = [apply_color_perm_grid(g, perm) for g in outs]
                p_tst = apply_color_perm_grid(tst, perm)
                tag = tuple(int(v) for v in perm)
            else:
                p_ins, p_outs, p_tst, tag = ins, outs, tst, None
            if len(p_ins) != len(p_outs):
                raise ValueError("train inputs and outputs differ in number")
            toks: list[int] = []
            for gi, go in zip(p_ins, p_outs):
                toks += encode_example(gi, go)
            toks += encode_example(p_tst, None)
            pos = compute_positions_3d(toks)
            for _ in range(max(1, num_samples)):
                prompts.append(toks)
                positions.append(pos)
                info.append((d_idx, tag))
    return prompts, positions, info


def augmented_constraints(task: dict, test_idx: int, info):
    """Per-variant colour palettes and output shapes for constrained decoding
    (src/inference.py:236-282, 798-808): the palette is the set of colours in the train pairs mapped
    through the variant's colour permutation; the shape is the train outputs' common shape (if any),
    transposed for the dihedral transforms that swap height and width."""
    colours: set[int] = set()
    for pair in task.get("train", []):
        for key in ("input", "output"):
            grid = pair.get(key)
            if grid is not None:
                colours.update(int(v) for row in grid for v in row)
    shapes_seen = []
    for pair in task.get("train", []):
        g = pair.get("output")
        if not g or not g[0] or any(len(row) != len(g[0]) for row in g):
            shapes_seen = None
            break
        shapes_seen.append((len(g), len(g[0])))
    base_shape = shapes_seen[0] if shapes_seen and all(s == shapes_seen[0] for s in shapes_seen) else None
    palettes, shapes = [], []
    for d_idx, perm in info:
        palettes.append(colours if perm is None else {int(perm[c]) for c in colours})
        if base_shape is None:
            shapes.append(None)
        else:
            shapes.append((base_shape[1], base_shape[0]) if d_idx in (1, 3, 6, 7) else base_shape)
    return palettes, shapes


def chunk_constraints(palettes, shapes, palette_penalty: float, shape_penalty: float) -> DecodingConstraints:
    """DecodingConstraints of one chunk, built like the reference does (src/inference.py:842-875)."""
    n = len(palettes)
    palette_mask = None
    if any(palettes):
        m = torch.ones((n, 10), dtype=torch.bool)
        for i, pal in enumerate(palettes):
            if pal:
                m[i] = False
                for c in pal:
                    if 0 <= c < 10:
                        m[i, c] = True
        palette_mask = m
    target_shape = None
    if any(s is not None for s in shapes):
        t = torch.full((n, 2), -1, dtype=torch.long)
        for i, s in enumerate(shapes):
            if s is not None:
                t[i, 0], t[i, 1] = s[0], s[1]
        target_shape = t
    return DecodingConstraints(palette_mask=palette_mask, target_shape=target_shape,
                               palette_penalty=palette_penalty, shape_penalty=shape_penalty)


def pad_prompts(prompts, positions, left: bool = True):
    """Pad ragged prompts to one length with END / (0,0,0) (src/inference.py:878-890)."""
    n = len(prompts)
    width = max(len(p) for p in prompts)
    ids = np.full((n, width), END_TOKEN_ID, dtype=np.int64)
    pos = np.zeros((n, width, 3), dtype=np.int64)
    mask = np.zeros((n, width), dtype=bool)
    for i, (p, q) in enumerate(zip(prompts, positions)):
        k = len(p)
        sl = slice(width - k, width) if left else slice(0, k)
        ids[i, sl] = p
        pos[i, sl] = q
        mask[i, sl] = True
    return ids, pos, mask


def predict_with_augmentations(model, task: dict, test_idx: int, device, example_id: int = 0,
                               use_train_examples: bool = True, num_color_perms: int = 8,
                               max_output_tokens: int = 900, num_samples: int = 1,
                               sample_temperature: float = 0.0, sample_top_k: int | None = None,
                               constrain_decoding: bool = False, palette_penalty: float = 2.0,
                               shape_penalty: float = 2.0, batched: bool = True, use_compile: bool = False,
                               max_batch_size: int = 16, merge_chunks: bool = True,
                               freeze_finished: bool = True):
    """Candidates under all augmentations for AAIVR voting (``src/inference.py:697-920``).

    Returns ``[(grid | None, dihedral_idx, colour_perm | None), ...]`` in the reference's order.
    Prompts are laid out in chunks of ``max_batch_size`` left-padded rows exactly as the reference's
    batched path does, so each chunk reproduces its semantics (including which hidden state yields
    the first token of a left-padded row); with ``merge_chunks`` the chunks share one session
    (one prefill, one decode loop for all of them) instead of one ``generate_output`` call each.

    A row that has emitted END is frozen here; the reference keeps decoding it until every row of its
    16-row chunk has finished and reads the grid after the LAST IO_SEP of the row, so a finished row
    that later emits another IO_SEP yields a different candidate there.  For exactly the reference's
    candidates pass ``freeze_finished=False`` together with ``merge_chunks=False`` (one call per chunk,
    each stopping when its own 16 rows have finished).
    """
    device = torch.device(device)
    engine = _resolve_engine(model, device)
    prompts, positions, info = build_augmented_prompts(task, test_idx, use_train_examples,
                                                       num_color_perms, num_samples)
    palettes = shapes = None
    if constrain_decoding:
        palettes, shapes = augmented_constraints(task, test_idx, info)
    if not batched:
        # The reference's sequential path runs every variant alone and unpadded
        # (src/inference.py:923-1003).  A right-padded batch gives each row exactly that (its keys,
        # its last token), so all variants share one session unless max_seq_len would cut some
        # rows shorter than others, in which case they run one by one.
        lens = [len(p) for p in prompts]
        out = []
        if lens and max(lens) + max_output_tokens <= engine.max_seq_len:
            ids, pos, mask = pad_prompts(prompts, positions, left=False)
            n = len(prompts)
            cons = None
            if constrain_decoding:
                cons = _constraints_dict(chunk_constraints(palettes, shapes, palette_penalty, shape_penalty), n)
            seed = int(torch.randint(0, 2 ** 62, (1,)).item()) if sample_temperature > 0 else 0
            trace = generate_tokens(engine, ids, pos, mask, np.full(n, example_id, dtype=np.int64),
                                    max_output_tokens, stop_on_end=True, constraints=cons,
                                    temperature=float(sample_temperature), top_k=sample_top_k, sample_seed=seed,
                                    freeze_finished=freeze_finished)
            gen = trace.tokens.cpu().tolist()
            for i, (d_idx, tag) in enumerate(info):
                out.append((_grid_after_last_sep([int(t) for t in prompts[i]] + gen[i]), d_idx, tag))
            return out
        for i, (d_idx, tag) in enumerate(info):
            cons = None
            if constrain_decoding:
                cons = chunk_constraints(palettes[i:i + 1], shapes[i:i + 1], palette_penalty, shape_penalty)
            ids_t = torch.tensor([[int(t) for t in prompts[i]]], dtype=torch.long, device=device)
            full = generate_output(engine, ids_t, torch.from_numpy(np.asarray(positions[i])[None]).to(device),
                                   torch.tensor([example_id], dtype=torch.long, device=device),
                                   max_new_tokens=max_output_tokens, temperature=sample_temperature,
                                   top_k=sample_top_k, stop_on_end=True, constraints=cons,
                                   freeze_finished=freeze_finished)
            out.append((_grid_after_last_sep(full[0].cpu().tolist()), d_idx, tag))
        return out
    chunks = [slice(c0, min(c0 + max_batch_size, len(prompts))) for c0 in range(0, len(prompts), max_batch_size)]
    padded = [pad_prompts(prompts[c], positions[c], left=True) for c in chunks]
    width = max((p[0].shape[1] for p in padded), default=0)
    out = []
    if merge_chunks and len(chunks) > 1 and width + max_output_tokens <= engine.max_seq_len:
        # All chunks in ONE session.  Each chunk keeps its own left-padded layout (what decides which
        # hidden state yields a row's first token, src/inference.py:420-423); the narrower chunks
        # get masked columns on the right, which changes neither a row's valid keys nor the padded
        # index len - 1.  No chunk is clamped by max_seq_len here, so every row may generate
        # max_output_tokens as it would in its own chunk.
        n = len(prompts)
        ids = np.full((n, width), END_TOKEN_ID, dtype=np.int64)
        pos = np.zeros((n, width, 3), dtype=np.int64)
        mask = np.zeros((n, width), dtype=bool)
        for c, (ci, cp, cm) in zip(chunks, padded):
            w = ci.shape[1]
            ids[c, :w], pos[c, :w], mask[c, :w] = ci, cp, cm
        cons = None
        if constrain_decoding:
            cons = _constraints_dict(chunk_constraints(palettes, shapes, palette_penalty, shape_penalty), n)
        seed = int(torch.randint(0, 2 ** 62, (1,)).item()) if sample_temperature > 0 else 0
        trace = generate_tokens(engine, ids, pos, mask, np.full(n, example_id, dtype=np.int64), max_output_tokens,
                                stop_on_end=True, constraints=cons, temperature=float(sample_temperature),
                                top_k=sample_top_k, sample_seed=seed, freeze_finished=freeze_finished)
        gen = trace.tokens.cpu().tolist()
        for i, (d_idx, tag) in enumerate(info):
            # the reference reads the grid after the last IO_SEP of padding + prompt + generated
            # tokens (src/inference.py:906-915); the padding (END tokens before the prompt) plays no part
            out.append((_grid_after_last_sep([int(t) for t in prompts[i]] + gen[i]), d_idx, tag))
        return out
    for c, (ids, pos, mask) in zip(chunks, padded):
        ids_t = torch.from_numpy(ids).to(device)
        cons = None
        if constrain_decoding:
            cons = chunk_constraints(palettes[c], shapes[c], palette_penalty, shape_penalty)
        full = generate_output(engine, ids_t, torch.from_numpy(pos).to(device),
                               torch.full((ids.shape[0],), example_id, dtype=torch.long, device=device),
                               attention_mask=torch.from_numpy(mask).to(device),
                               max_new_tokens=max_output_tokens, temperature=sample_temperature,
                               top_k=sample_top_k, stop_on_end=True, constraints=cons,
                               freeze_finished=freeze_finished)
        rows = full.cpu().tolist()
        for i, toks in enumerate(rows):
            d_idx, tag = info[c.start + i]
            out.append((_grid_after_last_sep(toks), d_idx, tag))
    return out
