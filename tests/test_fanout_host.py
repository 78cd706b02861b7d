"""Host side of the device fan-out (no GPU): variant enumeration and prompt lengths from grid
shapes alone, and the vote taken from candidate records, against the oracle and the loop codec."""
import random

import numpy as np
import torch

from mdlarc_scale_b200 import fanout, sharding, synthetic
from mdlarc_scale_b200.inference import build_augmented_prompts
from oracle import arc_fanout, arc_tokens, arc_vote


def _tasks(seed=4, n=5):
    tasks = synthetic.capped_tasks(seed, n, 1, 3, 1, 7, None)
    tasks[0]["test"].append({"input": [[1, 2, 3]]})          # a task with two test inputs
    tasks[1]["train"][0]["input"] = [[5]]                     # 1 x 1 grid
    return tasks


def test_variant_table_matches_loop_enumeration():
    tasks = _tasks()
    table = fanout.TaskTable(tasks, "cpu", num_color_perms=4)
    vt = table.variants()
    ref = sharding.enumerate_variants(tasks, num_color_perms=4)
    assert len(vt) == len(ref)
    for i, v in enumerate(ref):
        assert (vt.task[i], vt.test_idx[i], vt.dihedral[i]) == (v.task, v.test_idx, v.dihedral)
        assert table.perm_tuple(int(vt.perm[i])) == v.perm
        assert vt.length[i] == len(v.tokens)
        toks, pos = arc_fanout.variant_prompt(tasks[v.task], v.test_idx, v.dihedral, v.perm)
        assert toks == list(v.tokens) and np.array_equal(pos, v.positions)


def test_oracle_prompt_matches_reference_order(golden_tokens):
    """The oracle's variant prompt uses the pinned codec, dihedral and permutation primitives."""
    c = golden_tokens["cases"][0]
    task = {"train": [{"input": c["input"], "output": c["output"]}], "test": [{"input": c["output"]}]}
    toks, pos = arc_fanout.variant_prompt(task, 0, 0, None)
    assert toks == c["tokens"] and pos.tolist() == c["positions"]
    prompts, positions, info = build_augmented_prompts(task, 0, True, 3, 1)
    perms = arc_tokens.color_permutations(3, seed=42)
    for p, q, (d, perm) in zip(prompts, positions, info):
        want_t, want_p = arc_fanout.variant_prompt(task, 0, d, perm)
        assert list(p) == want_t and np.array_equal(np.asarray(q), want_p)
        assert perm is None or perm in [tuple(int(v) for v in r) for r in perms]


def test_malformed_tasks_are_rejected():
    import pytest
    bad = {"train": [{"input": [[1, 2], [3]], "output": [[1]]}], "test": [{"input": [[1]]}]}
    with pytest.raises(ValueError):
        fanout.TaskTable([bad], "cpu")
    bad2 = {"train": [], "test": [{"input": [[11]]}]}
    with pytest.raises(ValueError):
        fanout.TaskTable([bad2], "cpu")


def _random_generation(rng, grid, d, perm, max_new):
    """Tokens a model might emit for a variant: the transformed grid, sometimes damaged."""
    g = arc_tokens.dihedral(grid, d)
    if perm is not None:
        g = [[int(perm[c]) for c in row] for row in g]
    toks = arc_tokens.grid_to_tokens(g) + [arc_tokens.END]
    kind = rng.random()
    if kind < 0.1:
        toks = [arc_tokens.END]                                   # nothing
    elif kind < 0.2 and len(toks) > 3:
        del toks[int(rng.integers(0, len(toks) - 2))]             # usually jagged
    elif kind < 0.3:
        toks = [1, 2, arc_tokens.IO_SEP] + toks                   # a second IO_SEP: the grid restarts
    elif kind < 0.4:
        toks = [arc_tokens.NEWLINE, arc_tokens.START] + toks      # ignored tokens
    elif kind < 0.45:
        toks = [arc_tokens.NEWLINE, arc_tokens.NEWLINE, arc_tokens.END]   # only separators
    elif kind < 0.5:
        toks = toks[:-1]                                          # END never emitted
    toks = toks[:max_new]
    tail = rng.integers(0, 14, size=max_new - len(toks)).tolist() if arc_tokens.END in toks else \
        [arc_tokens.NEWLINE] * (max_new - len(toks))
    return toks + tail


def make_generations(tasks, table, vt, max_new, seed=0):
    rng = np.random.default_rng(seed)
    rows = np.zeros((len(vt), max_new), np.int32)
    for i in range(len(vt)):
        task = tasks[int(vt.task[i])]
        # half the variants agree on one answer, the rest on the test input (input copies) or noise
        pick = rng.random()
        if pick < 0.5:
            grid = task["train"][0]["output"]
        elif pick < 0.7:
            grid = task["test"][int(vt.test_idx[i])]["input"]
        else:
            grid = synthetic.random_grid(rng, 1, 5)
        perm = table.perm_tuple(int(vt.perm[i]))
        if pick >= 0.5 and pick < 0.6:
            # an input copy in the variant's own frame is not one in the task's frame unless d = 0, perm = None
            rows[i] = _random_generation(rng, grid, 0, None, max_new)
        else:
            rows[i] = _random_generation(rng, grid, int(vt.dihedral[i]), perm, max_new)
    return rows


def host_records(tasks, table, vt, rows):
    rec = np.zeros((len(vt), fanout.RECORD_BYTES), np.uint8)
    for i in range(len(vt)):
        test_input = tasks[int(vt.task[i])]["test"][int(vt.test_idx[i])]["input"]
        rec[i] = np.frombuffer(arc_fanout.candidate_record(rows[i], int(vt.dihedral[i]),
                                                           table.perm_tuple(int(vt.perm[i])), test_input), np.uint8)
    return rec


def test_vote_from_records_equals_vote_from_tokens():
    tasks = _tasks(seed=9, n=6)
    table = fanout.TaskTable(tasks, "cpu", num_color_perms=5)
    vt = table.variants()
    max_new = 48
    rows = make_generations(tasks, table, vt, max_new, seed=3)
    rec = host_records(tasks, table, vt, rows)
    status = fanout.record_fields(rec)[0]
    assert {0, 1, 2} <= set(status.tolist())                       # all three kinds occur
    assert fanout.record_fields(rec)[1].sum() > 0                  # and some input copies
    got = fanout.vote_records(rec, vt, top_k=2, seed=7)
    variants = sharding.enumerate_variants(tasks, num_color_perms=5)
    cands = sharding.candidates_from_tokens(variants, rows, np.arange(len(vt)))
    want = sharding.vote_all(tasks, cands, top_k=2, seed=7)
    assert got == want
    for (ti, te), preds in cands.items():                          # and the oracle's vote
        o = arc_vote.aaivr_predict(preds, 2, tasks[ti]["test"][te]["input"], rng=random.Random(7 + 1000003 * ti + te))
        assert got[(ti, te)] == o
    keep = fanout.vote_records(rec, vt, top_k=3, seed=1, discard_input_copies=False)
    for (ti, te), preds in cands.items():
        o = arc_vote.aaivr_predict(preds, 3, tasks[ti]["test"][te]["input"], discard_input_copies=False,
                                   rng=random.Random(1 + 1000003 * ti + te))
        assert keep[(ti, te)] == o


def test_tally_of_empty_and_invalid_groups():
    """No valid candidate for a test input gives an empty vote (tests/test_voting.py:194-233)."""
    tasks = _tasks(seed=9, n=3)
    table = fanout.TaskTable(tasks, "cpu", num_color_perms=2)
    vt = table.variants()
    rows = make_generations(tasks, table, vt, 32, seed=1)
    rec = host_records(tasks, table, vt, rows)
    first = vt.template == 0
    rec[first, 0] = np.where(np.arange(first.sum()) % 2 == 0, 0, 2)     # nothing / malformed only
    tallies = fanout.tally_records(rec, vt)
    ranked, n_total, n_valid = tallies[(0, 0)]
    assert ranked(random.Random(0)) == [] and n_total == 16 and n_valid == 0
    assert fanout.vote_records(rec, vt)[(0, 0)] == []
    assert fanout.vote_records(np.zeros((0, fanout.RECORD_BYTES), np.uint8),
                               fanout.TaskTable([], "cpu").variants()) == {}
