"""Fan-out kernels against the oracle, bit for bit: prompts of every (dihedral x colour permutation)
variant built on the device, candidate records from generated tokens, and the sharded pipeline that
uses both against the host-side pipeline."""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import have_b200
from oracle import arc_fanout
from test_fanout_host import _tasks, host_records, make_generations

pytestmark = pytest.mark.gpu


def _need_gpu():
    if not have_b200():
        pytest.fail("these tests need a B200 (compute capability 10.x)")


def _big_tasks():
    from mdlarc_scale_b200 import synthetic
    tasks = _tasks(seed=11, n=4)
    tasks += synthetic.capped_tasks(12, 2, 2, 3, 24, 30, None)      # large grids: positions clamp at y = 29
    tasks.append({"train": [{"input": [[1] * 30 for _ in range(30)], "output": [[2] * 30 for _ in range(30)]}],
                  "test": [{"input": [[3, 0, 4]]}]})
    tasks.append({"train": [], "test": [{"input": [[7], [8]]}]})    # no train pairs
    return tasks


def test_device_prompts_equal_oracle_prompts():
    _need_gpu()
    from mdlarc_scale_b200 import fanout
    tasks = _big_tasks()
    table = fanout.TaskTable(tasks, "cuda:0", num_color_perms=5)
    vt = table.variants()
    rng = np.random.default_rng(0)
    idx = rng.permutation(len(vt))                      # any order, any subset
    for sel in (idx[:7], idx, np.arange(len(vt))):
        rows = np.arange(len(sel))[::-1].copy()         # arbitrary cache rows
        plan = table.build_prompts(vt, sel, rows)
        fanout.check_status(plan)
        tok, pos = plan.token_ids.cpu().numpy(), plan.pos_xyz.cpu().numpy()
        seq, slot = plan.seq.cpu().numpy(), plan.kv_slot.cpu().numpy()
        cnt, kvr = plan.kv_count.cpu().numpy(), plan.kv_row.cpu().numpy()
        first = plan.first_row.cpu().numpy()
        o = 0
        for k, v in enumerate(sel.tolist()):
            want_t, want_p = arc_fanout.variant_prompt(tasks[int(vt.task[v])], int(vt.test_idx[v]),
                                                       int(vt.dihedral[v]), table.perm_tuple(int(vt.perm[v])))
            n = len(want_t)
            assert n == vt.length[v]
            assert tok[o: o + n].tolist() == want_t, (k, v)
            assert np.array_equal(pos[o: o + n], want_p), (k, v)
            assert (seq[o: o + n] == rows[k]).all()
            assert np.array_equal(slot[o: o + n], np.arange(n)) and np.array_equal(cnt[o: o + n], np.arange(n) + 1)
            assert np.array_equal(kvr[o: o + n], np.arange(o, o + n))
            o += n
            assert first[k] == o - 1
        assert o == plan.n_tokens == plan.n_kv_rows


def test_device_prompt_length_mismatch_is_reported():
    _need_gpu()
    from mdlarc_scale_b200 import fanout
    tasks = _tasks(seed=2, n=2)
    table = fanout.TaskTable(tasks, "cuda:0", num_color_perms=2)
    vt = table.variants()
    vt.length = vt.length.copy()
    vt.length[3] += 1                                    # host and device disagree about one prompt
    plan = table.build_prompts(vt, np.arange(len(vt)), np.arange(len(vt)))
    with pytest.raises(RuntimeError):
        fanout.check_status(plan)


def test_candidate_records_equal_oracle_records():
    _need_gpu()
    from mdlarc_scale_b200 import fanout
    tasks = _tasks(seed=9, n=6)
    table = fanout.TaskTable(tasks, "cuda:0", num_color_perms=5)
    vt = table.variants()
    for max_new, seed in ((48, 3), (931, 4)):
        rows = make_generations(tasks, table, vt, max_new, seed=seed)
        if max_new == 931:
            rows[0] = ([1] * 30 + [11]) * 30 + [13]     # the largest grid the token budget allows
            rows[1] = [5] * 931                          # one row of 931 cells, END never emitted
            rows[2] = [5, 11] * 465 + [13]               # 465 rows of one cell
        want = host_records(tasks, table, vt, rows)
        idx = np.arange(len(vt))
        idx_pad = np.concatenate([idx, [-1, -1]])        # padding rows of an uneven shard
        toks = torch.from_numpy(np.concatenate([rows, np.full((2, max_new), 13, np.int32)])).cuda()
        rec = torch.full((len(idx_pad), fanout.RECORD_BYTES), 255, dtype=torch.uint8, device="cuda")
        table.canonicalize(toks, vt, idx_pad, rec)
        got = rec.cpu().numpy()
        assert np.array_equal(got[: len(vt)], want)
        assert not got[len(vt):].any()
        st = fanout.record_fields(got)[0]
        assert {0, 1, 2} <= set(st.tolist())


def test_fanout_argument_errors():
    _need_gpu()
    from mdlarc_scale_b200 import _lib
    lib = _lib.load()
    a = _lib.CandidateArgs(n_rows=1, max_new=1000, n_perms=1)
    assert lib.arcb_canonicalize_candidates(C.byref(a), None) == _lib.E_ARG
    assert b"max_new" in lib.arcb_last_error()
    b = _lib.PromptBuildArgs(n_variants=1, n_perms=1)
    assert lib.arcb_build_prompts(C.byref(b), None) == _lib.E_ARG
    assert lib.arcb_build_prompts(None, None) == _lib.E_ARG


def test_sharded_records_pipeline_equals_host_pipeline():
    _need_gpu()
    from mdlarc_scale_b200 import fanout, sharding, synthetic
    from mdlarc_scale_b200.engine import Engine
    cfg, sd = synthetic.seeded_weights("tiny", 0, 8.0)
    eng = Engine(sd, cfg, "cuda:0")
    tasks = synthetic.capped_tasks(5, 3, 1, 2, 1, 6, None)
    max_new = 32
    table = fanout.TaskTable(tasks, eng.device, num_color_perms=3)
    vt = table.variants()
    variants = sharding.enumerate_variants(tasks, num_color_perms=3)
    # one wave each way: identical packed batches, so identical tokens, records and votes
    rec = sharding.generate_sharded_records(table, vt, max_new, 0, 1, eng, wave_size=len(vt))
    buf = sharding.generate_sharded(variants, max_new, 0, 1, sharding.engine_wave_fn(eng), eng.device,
                                    wave_size=len(variants)).cpu().numpy()
    layout = sharding.gather_layout([len(v.tokens) for v in variants], 1)
    rows = np.zeros_like(buf)
    rows[layout] = buf                                   # back to variant order
    want = host_records(tasks, table, vt, rows)
    assert np.array_equal(rec, want)
    cands = sharding.candidates_from_tokens(variants, buf, layout)
    assert fanout.vote_records(rec, vt, 2, seed=7) == sharding.vote_all(tasks, cands, top_k=2, seed=7)
    # several waves and several prefill calls per wave: complete, well-formed records
    rec2 = sharding.generate_sharded_records(table, vt, max_new, 0, 1, eng, wave_size=20, max_prefill_tokens=600)
    st = fanout.record_fields(rec2)[0]
    assert st.shape == (len(vt),) and set(st.tolist()) <= {0, 1, 2}
    assert (fanout.record_fields(rec2)[4] >= 1).all()
    eng.close()
