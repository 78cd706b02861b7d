"""Multi-GPU partition of the augmentation fan-out: shard (task x dihedral x colour-permutation x
sample) variants over ranks, generate locally, ONE all-gather of the decoded candidates, vote.

The reference shards whole tasks (``src/eval.py:569-571``) and all-reduces six scalars
(``src/eval.py:1203-1208``).  Here every variant is an independent sequence until the vote, so
variants are dealt to ranks by length-sorted round-robin (balances tokens, keeps each rank's
length buckets tight).  The assignment is a pure function of the prompt lengths, so every rank
knows which variant sits in which row of the gathered buffer and nothing but tokens is sent:
each rank's decode kernels write their tokens straight into that rank's slice of the gather
buffer (no pack/copy kernel), and a single in-place ``all_gather_into_tensor`` completes it.
Votes are then computed identically on every rank, in the reference's candidate order with a
seeded tie-break rng, so no result broadcast is needed.
"""
from __future__ import annotations

import random
from dataclasses import dataclass

import numpy as np
import torch

from .data import END_TOKEN_ID, IO_SEP_TOKEN_ID
from .inference import _grid_after_last_sep, build_augmented_prompts, pad_prompts
from .voting import aaivr_predict


@dataclass
class Variant:
    task: int          # index into the task list
    test_idx: int
    dihedral: int
    perm: tuple | None
    tokens: list       # prompt tokens
    positions: np.ndarray


def enumerate_variants(tasks: list[dict], num_color_perms: int = 8, num_samples: int = 1,
                       use_train_examples: bool = True) -> list[Variant]:
    """All variants of all (task, test input) pairs in canonical order: task, test index, then the
    reference's candidate order (dihedral-major, permutation, sample; src/inference.py:794-827)."""
    out: list[Variant] = []
    for ti, task in enumerate(tasks):
        for test_idx in range(len(task["test"])):
            prompts, positions, info = build_augmented_prompts(task, test_idx, use_train_examples,
                                                               num_color_perms, num_samples)
            for p, q, (d, perm) in zip(prompts, positions, info):
                out.append(Variant(ti, test_idx, d, perm, p, q))
    return out


def assign(lengths, world: int) -> list[np.ndarray]:
    """Variant indices of each rank: sort by prompt length (stable), deal round-robin."""
    order = np.argsort(np.asarray(lengths), kind="stable")
    return [order[r::world] for r in range(world)]


def rows_per_rank(n_variants: int, world: int) -> int:
    return (n_variants + world - 1) // world


def gather_layout(lengths, world: int) -> np.ndarray:
    """variant id held by each row of the gathered buffer ([world * rows_per_rank], -1 = padding)."""
    n = len(lengths)
    per = rows_per_rank(n, world)
    ids = np.full(world * per, -1, dtype=np.int64)
    for r, mine in enumerate(assign(lengths, world)):
        ids[r * per: r * per + len(mine)] = mine
    return ids


def generate_sharded(variants: list[Variant], max_new: int, rank: int, world: int, generate_wave,
                     device, group=None, wave_size: int = 1024) -> torch.Tensor:
    """Generate this rank's variants in waves and all-gather every rank's tokens.

    ``generate_wave(ids, pos, mask, out_tokens)`` must fill ``out_tokens`` (int32 view
    ``[n, max_new]`` of the gather buffer, pre-filled with END) with the generated tokens of the
    right-padded batch ``ids/pos/mask``.  Returns the gathered int32 ``[world * per, max_new]``.
    """
    lengths = [len(v.tokens) for v in variants]
    per = rows_per_rank(len(variants), world)
    buf = torch.full((world * per, max_new), END_TOKEN_ID, dtype=torch.int32, device=device)
    mine = assign(lengths, world)[rank]
    local = buf[rank * per: (rank + 1) * per]
    for w0 in range(0, len(mine), wave_size):
        idx = mine[w0: w0 + wave_size]
        ids, pos, mask = pad_prompts([variants[i].tokens for i in idx], [variants[i].positions for i in idx],
                                     left=False)
        generate_wave(ids, pos, mask, local[w0: w0 + len(idx)])
    if world > 1:
        import torch.distributed as dist
        dist.all_gather_into_tensor(buf, local, group=group)  # in place: `local` is this rank's slice
    return buf


def candidates_from_tokens(variants: list[Variant], gathered: np.ndarray, layout: np.ndarray):
    """Per (task, test_idx): candidate tuples in canonical order from the gathered token rows."""
    row_of = np.full(len(variants), -1, dtype=np.int64)
    valid = layout >= 0
    row_of[layout[valid]] = np.flatnonzero(valid)
    out: dict[tuple[int, int], list] = {}
    for vid, v in enumerate(variants):
        gen = gathered[row_of[vid]].tolist()
        if END_TOKEN_ID in gen:
            gen = gen[: gen.index(END_TOKEN_ID) + 1]
        # the prompt ends with IO_SEP; the grid is read after the last IO_SEP (src/inference.py:908-911)
        grid = _grid_after_last_sep([IO_SEP_TOKEN_ID] + gen)
        out.setdefault((v.task, v.test_idx), []).append((grid, v.dihedral, v.perm))
    return out


def vote_all(tasks: list[dict], candidates: dict, top_k: int = 2, seed: int = 0) -> dict:
    """AAIVR top-k per (task, test_idx); tie-breaks from ``random.Random(seed + 1000003 * task + test_idx)``."""
    out = {}
    for (ti, test_idx), preds in sorted(candidates.items()):
        rng = random.Random(seed + 1000003 * ti + test_idx)
        out[(ti, test_idx)] = aaivr_predict(preds, top_k=top_k, test_input=tasks[ti]["test"][test_idx]["input"],
                                            rng=rng)
    return out


def engine_wave_fn(engine, stop_on_end: bool = True, max_prefill_tokens: int = 65536):
    """``generate_wave`` backed by the B200 engine: the session's token output IS the gather-buffer slice."""
    from .engine import chunk_rows, plan_prefill

    def run(ids, pos, mask, out_tokens):
        lens = mask.sum(axis=1)
        n, max_new = out_tokens.shape
        cap = max(int(min(max_prefill_tokens, int(lens.sum()) + 2 * n)), int(lens.max()) + 2, n)
        sess = engine.new_session(n, int(lens.max()) + max_new, max_new, cap, stop_on_end=stop_on_end,
                                  out_tokens=out_tokens)
        for rows in chunk_rows(lens, cap):
            sess.prefill(plan_prefill(ids, pos, mask, rows).to(engine.device), None)
        done = 0
        while done < max_new - 1:
            k = min(32, max_new - 1 - done)
            sess.decode(k)
            done += k
            if stop_on_end and sess.poll() >= n:
                break
        sess.poll()
        sess.close()

    return run


# ---------------------------------------------------------------------------
# the same pipeline with the fan-out on the device (fanout.TaskTable): prompts are built by a
# kernel from per-variant metadata, candidates leave as canonical records, and the records --
# a quarter of the size of the token rows -- are what the all-gather carries
# ---------------------------------------------------------------------------
def generate_sharded_records(table, vt, max_new: int, rank: int, world: int, engine, group=None,
                             wave_size: int = 1024, stop_on_end: bool = True,
                             max_prefill_tokens: int = 65536, example_ids=None, constraints: dict | None = None,
                             temperature: float = 0.0, top_k: int = 0, sample_seed: int = 0,
                             max_seq_len: int | None = None, gather: bool = True, timing: dict | None = None):
    """Generate this rank's variants and return every variant's candidate record in canonical
    variant order (uint8 ``[len(vt), RECORD_BYTES]``, identical on all ranks).

    ``example_ids`` (int array per variant) selects the example embedding of each sequence
    (``None`` = no example embedding).  ``constraints`` holds per-variant ``palette_mask``
    ``[n, 10]`` / ``target_shape`` ``[n, 2]`` arrays (either may be None) plus the scalar fields of
    ``inference._constraints_dict``.  ``max_seq_len`` caps prompt + generated tokens of a wave
    (src/inference.py:534-535, applied to the wave's longest prompt).
    """
    from .fanout import RECORD_BYTES, check_status
    dev = engine.device
    n_var = len(vt)
    per = rows_per_rank(n_var, world)
    mine = assign(vt.length, world)[rank]
    rec = torch.zeros((world * per, RECORD_BYTES), dtype=torch.uint8, device=dev)
    local = rec[rank * per: (rank + 1) * per]
    for w0 in range(0, len(mine), wave_size):
        idx = mine[w0: w0 + wave_size]
        n = len(idx)
        lens = vt.length[idx]
        new = max_new if max_seq_len is None else min(max_new, int(max_seq_len) - int(lens.max()))
        if new <= 0:
            continue   # no room to generate: these variants keep status 0 (no grid)
        tokens = torch.full((n, new), END_TOKEN_ID, dtype=torch.int32, device=dev)
        cap = max(int(min(max_prefill_tokens, int(lens.sum()))), int(lens.max()), n)
        wave_cons = None
        if constraints is not None:
            wave_cons = dict(constraints)
            for key in ("palette_mask", "target_shape"):
                if constraints.get(key) is not None:
                    wave_cons[key] = np.ascontiguousarray(constraints[key][idx])
        sess = engine.new_session(n, int(lens.max()) + new, new, cap, stop_on_end=stop_on_end,
                                  out_tokens=tokens, constraints=wave_cons, temperature=temperature,
                                  top_k=top_k, sample_seed=sample_seed, sample_stream=idx)
        ex = None
        if example_ids is not None:
            ex = torch.from_numpy(np.ascontiguousarray(np.asarray(example_ids)[idx], dtype=np.int32)).to(dev)
        plans, c0, tot = [], 0, 0
        for i in range(n + 1):   # greedy split into prefill calls of at most `cap` packed tokens
            if i == n or tot + int(lens[i]) > cap:
                rows = np.arange(c0, i)
                plans.append(table.build_prompts(vt, idx[rows], rows))
                sess.prefill(plans[-1], ex)
                c0, tot = i, 0
            if i < n:
                tot += int(lens[i])
        done = 0
        while done < new - 1:
            k = min(32, new - 1 - done)
            sess.decode(k)
            done += k
            if stop_on_end and sess.poll() >= n:
                break
        sess.poll()
        for p in plans:
            check_status(p)
        table.canonicalize(tokens, vt, idx, local[w0: w0 + n])   # straight into the gather slice
        sess.close()      # frees the wave's cache before the next wave allocates its own
        del sess, plans, tokens
    if not gather:
        return rec
    return gather_records(rec, rank, world, vt.length, group, timing)


def gather_records(rec: torch.Tensor, rank: int, world: int, lengths, group=None,
                   timing: dict | None = None) -> np.ndarray:
    """Complete the gather buffer ``rec`` (``[world * per, width]``, this rank's slice filled) with ONE
    in-place all-gather and return its rows in canonical variant order (host array)."""
    per = rec.shape[0] // world
    if world > 1:
        import torch.distributed as dist
        timed = timing is not None and rec.is_cuda
        if timed:
            # measurement only: line the ranks up first, so that the events bracket the collective
            # itself and not the wait for the slowest rank's generation
            torch.cuda.synchronize(rec.device)
            t_wait = __import__("time").perf_counter()
            dist.barrier(group=group)
            torch.cuda.synchronize(rec.device)
            timing["wait_for_slowest_rank_ms"] = (__import__("time").perf_counter() - t_wait) * 1e3
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        dist.all_gather_into_tensor(rec, rec[rank * per: (rank + 1) * per], group=group)
        if timed:
            e1.record()
            e1.synchronize()
            timing["all_gather_ms"] = e0.elapsed_time(e1)
    if timing is not None:
        timing.setdefault("all_gather_ms", 0.0)
        timing["gather_bytes"] = int(rec.numel() * rec.element_size())
    return records_in_variant_order(rec, lengths, world)


def records_in_variant_order(rec: torch.Tensor, lengths, world: int) -> np.ndarray:
    """Rows of a complete gather buffer re-ordered to canonical variant order (host array)."""
    layout = gather_layout(lengths, world)
    valid = layout >= 0
    out = np.zeros((len(lengths),) + tuple(rec.shape[1:]), rec.cpu().numpy().dtype)
    out[layout[valid]] = rec.cpu().numpy()[valid]
    return out
