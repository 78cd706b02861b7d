"""Variant sharding + single all-gather + vote on CPU ranks (gloo, world_size 2) with a stand-in
token generator: the gathered candidates and the votes must equal the single-process result."""
import os
import pickle
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from mdlarc_scale_b200 import sharding, synthetic  # noqa: E402
from mdlarc_scale_b200.data import grid_to_tokens  # noqa: E402

MAX_NEW = 40


def fake_wave(ids, pos, mask, out_tokens):
    """Deterministic stand-in for the GPU generator: emits a small grid that depends only on the
    prompt (so identical prompts vote together), then END."""
    for i in range(ids.shape[0]):
        toks = ids[i][mask[i]]
        h = 1 + int(toks.sum()) % 3
        w = 1 + int(len(toks)) % 4
        grid = [[int((toks[(r * w + c) % len(toks)] + r) % 10) for c in range(w)] for r in range(h)]
        gen = (grid_to_tokens(grid) + [13])[:MAX_NEW]
        out_tokens[i, :len(gen)] = torch.tensor(gen, dtype=torch.int32)


def _tasks():
    return synthetic.capped_tasks(77, 3, 1, 2, 1, 5, None)


def _run(rank, world, port, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        tasks = _tasks()
        variants = sharding.enumerate_variants(tasks, num_color_perms=3)
        buf = sharding.generate_sharded(variants, MAX_NEW, rank, world, fake_wave, "cpu", wave_size=7)
        layout = sharding.gather_layout([len(v.tokens) for v in variants], world)
        cands = sharding.candidates_from_tokens(variants, buf.numpy(), layout)
        votes = sharding.vote_all(tasks, cands, top_k=2, seed=3)
        # the records pipeline: this rank's candidates as canonical records in its slice of the
        # gather buffer (the CUDA path's kernel writes them; here the oracle does), one all-gather, vote
        from mdlarc_scale_b200 import fanout
        from oracle import arc_fanout
        table = fanout.TaskTable(tasks, "cpu", num_color_perms=3)
        vt = table.variants()
        per = sharding.rows_per_rank(len(vt), world)
        rec = torch.zeros((world * per, fanout.RECORD_BYTES), dtype=torch.uint8)
        for j, v in enumerate(sharding.assign(vt.length, world)[rank].tolist()):
            test_input = tasks[int(vt.task[v])]["test"][int(vt.test_idx[v])]["input"]
            rec[rank * per + j] = torch.frombuffer(bytearray(arc_fanout.candidate_record(
                buf[rank * per + j].tolist(), int(vt.dihedral[v]), table.perm_tuple(int(vt.perm[v])), test_input)),
                dtype=torch.uint8)
        records = sharding.gather_records(rec, rank, world, vt.length)
        votes_rec = fanout.vote_records(records, vt, top_k=2, seed=3)
        with open(f"{out_path}.{rank}", "wb") as f:
            pickle.dump((cands, votes, votes_rec), f)
    finally:
        dist.destroy_process_group()


def test_assign_is_balanced_and_complete():
    lengths = [5, 100, 7, 50, 60, 8, 9, 300, 2]
    parts = sharding.assign(lengths, 4)
    assert sorted(np.concatenate(parts).tolist()) == list(range(9))
    assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1
    layout = sharding.gather_layout(lengths, 4)
    assert len(layout) == 4 * 3 and sorted(layout[layout >= 0].tolist()) == list(range(9))


def test_candidate_order_matches_reference_enumeration():
    tasks = _tasks()
    variants = sharding.enumerate_variants(tasks, num_color_perms=3)
    assert len(variants) == 3 * 8 * 3
    first = [v for v in variants if v.task == 0]
    assert [v.dihedral for v in first] == [d for d in range(8) for _ in range(3)]
    assert first[0].perm is None and first[1].perm is not None and first[3].perm is None


def test_two_gloo_ranks_equal_single_process(tmp_path):
    tasks = _tasks()
    variants = sharding.enumerate_variants(tasks, num_color_perms=3)
    buf = sharding.generate_sharded(variants, MAX_NEW, 0, 1, fake_wave, "cpu", wave_size=7)
    layout = sharding.gather_layout([len(v.tokens) for v in variants], 1)
    want_c = sharding.candidates_from_tokens(variants, buf.numpy(), layout)
    want_v = sharding.vote_all(tasks, want_c, top_k=2, seed=3)
    assert any(len(v) > 0 for v in want_v.values())
    out = str(tmp_path / "res")
    port = 29500 + os.getpid() % 2000
    mp.spawn(_run, args=(2, port, out), nprocs=2, join=True)
    for r in range(2):
        with open(f"{out}.{r}", "rb") as f:
            cands, votes, votes_rec = pickle.load(f)
        assert cands == want_c
        assert votes == want_v
        assert votes_rec == want_v


def test_sampling_counter_streams_are_distinct_and_deal_never_shares_one():
    """The counter-based uniform number depends on (seed, stream id, position); stream ids are the
    job-wide variant numbers, so the length-sorted round-robin deal can never give two variants
    the same stream, whatever the number of ranks."""
    from mdlarc_scale_b200.engine import sample_uniform
    u = [sample_uniform(5, s, i) for s in range(64) for i in range(8)]
    assert all(0.0 <= x < 1.0 for x in u) and len(set(u)) == len(u)
    assert sample_uniform(5, 3, 2) == sample_uniform(5, 3, 2) != sample_uniform(6, 3, 2)
    assert abs(float(np.mean([sample_uniform(1, s, 0) for s in range(4096)])) - 0.5) < 0.02
    lengths = np.repeat(np.array([30, 30, 41, 17]), 4)          # 4 samples per prompt: equal lengths
    for world in (1, 2, 3, 4, 8):
        dealt = sharding.assign(lengths, world)
        ids = np.concatenate(dealt)
        assert sorted(ids.tolist()) == list(range(len(lengths)))      # each variant (= stream id) exactly once
