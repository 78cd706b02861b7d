"""Host side of the product (token codec, augmentation, voting, prefill planning) against the
reference's outputs (tests/golden) and the known answers of the reference's own tests."""
import random

import numpy as np
import pytest

from conftest import tuple_preds
from mdlarc_scale_b200 import data as D
from mdlarc_scale_b200 import voting as V


def test_special_ids():  # tests/test_data.py:97-106
    assert (D.VOCAB_SIZE, D.START_TOKEN_ID, D.NEWLINE_TOKEN_ID, D.IO_SEP_TOKEN_ID, D.END_TOKEN_ID) == (14, 10, 11, 12, 13)


def test_grid_to_tokens_kat():  # tests/test_data.py:108-113
    assert D.grid_to_tokens([[1, 2], [3, 4]]) == [1, 2, 11, 3, 4, 11]
    assert D.tokens_to_grid([1, 2, 11, 3, 4, 11]) == [[1, 2], [3, 4]]


def test_dihedral_kats():  # tests/test_data.py:267-300
    g = [[1, 2], [3, 4]]
    want = [[[1, 2], [3, 4]], [[3, 1], [4, 2]], [[4, 3], [2, 1]], [[2, 4], [1, 3]],
            [[2, 1], [4, 3]], [[3, 4], [1, 2]], [[1, 3], [2, 4]], [[4, 2], [3, 1]]]
    assert [f(g) for f in D.DIHEDRAL_TRANSFORMS] == want


def test_codec_positions_dihedral_golden(golden_tokens):
    for c in golden_tokens["cases"]:
        toks = D.encode_example(c["input"], c["output"]) + D.encode_example(c["output"], None)
        assert toks == c["tokens"]
        assert D.compute_positions_3d(toks).tolist() == c["positions"]
        assert [f(c["input"]) for f in D.DIHEDRAL_TRANSFORMS] == c["dihedral_in"]
        assert D.decode_output_grid(toks) == c["decoded"]
        for i in range(8):  # every inverse round-trips (tests/test_voting.py:48-101)
            assert V.invert_dihedral(D.DIHEDRAL_TRANSFORMS[i](c["input"]), i) == c["input"]
    for s, d in zip(golden_tokens["streams"], golden_tokens["decoded"]):
        assert D.decode_output_grid(s) == d
    long_row = [[1] * 40 for _ in range(35)]
    toks = D.encode_example(long_row, None)
    assert len(toks) == golden_tokens["long_n"]
    assert D.compute_positions_3d(toks)[-50:].tolist() == golden_tokens["long_positions_tail"]


def test_color_permutations(golden_tokens):
    assert D.generate_color_permutations(20, 42).tolist() == golden_tokens["perms20"]
    assert D.generate_color_permutations(3, 7).tolist() == golden_tokens["perms3_seed7"]
    p = D.generate_color_permutations(8)
    assert (p[:, 0] == 0).all() and (np.sort(p, axis=1) == np.arange(10)).all()
    assert V.invert_color_permutation(D.apply_color_perm_grid([[1, 2], [0, 9]], p[3]), tuple(p[3])) == [[1, 2], [0, 9]]


def test_color_inversion_kat():  # tests/test_voting.py:112-147
    perm = (0, 2, 1, 3, 4, 5, 6, 7, 8, 9)
    assert V.invert_color_permutation([[2, 1], [0, 3]], perm) == [[1, 2], [0, 3]]


def test_votes_golden(golden_votes):
    for c in golden_votes["cases"]:
        preds = tuple_preds(c["predictions"])
        votes = V.aggregate_votes(preds, test_input=c["test_input"], rng=random.Random(c["seed"]))
        assert [[g, n] for g, n in votes] == c["votes"]
        assert V.aaivr_predict(preds, 2, c["test_input"], rng=random.Random(c["seed"])) == c["top2"]
        assert V.aaivr_predict(preds, 3, c["test_input"], False, random.Random(c["seed"] + 100)) == c["top3_keep_copies"]
        assert V.compute_voting_stats(preds, test_input=c["test_input"]) == c["stats"]


def test_vote_edge_cases():  # tests/test_voting.py:194-203, 215-233
    assert V.aaivr_predict([]) == []
    assert V.aaivr_predict([(None, 0, None), (None, 3, None)]) == []
    a, b = [[1, 2], [3, 4]], [[5]]
    votes = V.aggregate_votes([(a, 0, None), (b, 0, None), (a, 0, None)], rng=random.Random(0))
    assert votes == [(a, 2), (b, 1)]
    rot = D.rot90(a)
    assert V.aggregate_votes([(a, 0, None), (rot, 1, None)], rng=random.Random(0)) == [(a, 2)]


def test_prefill_plan_right_and_left_padding():
    torch = pytest.importorskip("torch")
    from mdlarc_scale_b200.engine import chunk_rows, plan_prefill
    from mdlarc_scale_b200.inference import pad_prompts
    prompts = [[10, 1, 2, 11, 12], [10, 3, 11, 4, 11, 12, 5, 11]]
    positions = [D.compute_positions_3d(p) for p in prompts]
    for left in (False, True):
        ids, pos, mask = pad_prompts(prompts, positions, left=left)
        plan = plan_prefill(ids, pos, mask, np.arange(2))
        n_valid = 13
        if left:
            # row 0 has 5 tokens in width 8: index len-1 = 4 is a real token (3 pads precede it)
            assert plan.n_tokens == n_valid
            assert plan.first_row.tolist() == [1, 5 + 7]
        else:
            assert plan.n_tokens == n_valid
            assert plan.first_row.tolist() == [4, 12]
        assert plan.token_ids.tolist()[:5] == prompts[0]
        assert plan.kv_slot.tolist() == [0, 1, 2, 3, 4, 0, 1, 2, 3, 4, 5, 6, 7]
        assert plan.kv_count.tolist() == [1, 2, 3, 4, 5, 1, 2, 3, 4, 5, 6, 7, 8]
        assert plan.prompt_len.tolist() == [5, 8]
        # query blocks are listed most expensive first (the block whose last row sees the most keys)
        assert plan.qblock_row0.tolist() == [5, 0] and plan.qblock_rows.tolist() == [8, 5]
    # a left-padded row whose index len-1 falls in the padding gets a query-only row
    prompts = [[10, 12], [10, 3, 11, 4, 11, 12, 5, 11]]
    positions = [D.compute_positions_3d(p) for p in prompts]
    ids, pos, mask = pad_prompts(prompts, positions, left=True)
    plan = plan_prefill(ids, pos, mask, np.arange(2))
    assert plan.n_tokens == 11 and plan.kv_slot.tolist()[-1] == -1 and plan.kv_count.tolist()[-1] == 0
    assert plan.first_row.tolist() == [10, 9] and plan.token_ids.tolist()[-1] == 13
    assert plan.grid_in_output.tolist() == [0, 1]  # pad token END at z=0 -> not in output (reference quirk)
    assert [c.tolist() for c in chunk_rows(np.array([5, 8, 3]), 12)] == [[0], [1], [2]]
    assert [c.tolist() for c in chunk_rows(np.array([5, 8, 3]), 64)] == [[0, 1, 2]]


def test_no_cpu_fallback():
    torch = pytest.importorskip("torch")
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from mdlarc_scale_b200 import generate_output
    from oracle import arc_model as om

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.config = om.make_config("tiny")
            self.w = torch.nn.Parameter(torch.zeros(1))

    with pytest.raises(RuntimeError):
        generate_output(M(), torch.zeros(1, 4, dtype=torch.long), torch.zeros(1, 4, 3, dtype=torch.long))
    with pytest.raises(ValueError):
        generate_output(M(), torch.zeros(1, 4, dtype=torch.long), torch.zeros(1, 4, 3, dtype=torch.long),
                        attention_mask=torch.ones(2, 4, dtype=torch.bool))


def test_constraint_helpers_match_reference(golden_tokens):
    pytest.importorskip("torch")
    from mdlarc_scale_b200.inference import augmented_constraints, build_augmented_prompts, chunk_constraints
    task = golden_tokens["constraint_task"]
    _, _, info = build_augmented_prompts(task, 0, True, 3, 1)
    palettes, shapes = augmented_constraints(task, 0, info)
    rows = golden_tokens["constraint_rows"]
    assert len(rows) == len(info) == 24
    for row, (d, perm), pal, shp in zip(rows, info, palettes, shapes):
        assert d == row["dihedral"] and (perm is None) == (row["perm"] == 0)
        assert sorted(pal) == row["palette"]
        assert (list(shp) if shp else None) == row["shape"]
    cons = chunk_constraints(palettes[:5], shapes[:5], 2.0, 3.0)
    assert cons.palette_mask.shape == (5, 10) and cons.target_shape.shape == (5, 2)
    for i in range(5):
        assert sorted(cons.palette_mask[i].nonzero().flatten().tolist()) == sorted(palettes[i])
        assert cons.target_shape[i].tolist() == list(shapes[i])
    assert cons.palette_penalty == 2.0 and cons.shape_penalty == 3.0 and cons.disallow_tokens == (10, 12)


def test_vectorised_prompt_builder_equals_loop_version():
    pytest.importorskip("torch")
    from mdlarc_scale_b200 import inference, synthetic
    tasks = synthetic.capped_tasks(2, 4, 2, 4, 1, 30, 2048)
    for t in tasks:
        fast = inference.build_augmented_prompts(t, 0, True, 4, 2)
        saved = inference.as_rect_array
        inference.as_rect_array = lambda g: None   # forces the per-cell loop path
        try:
            slow = inference.build_augmented_prompts(t, 0, True, 4, 2)
        finally:
            inference.as_rect_array = saved
        assert fast[2] == slow[2] and len(fast[0]) == 8 * 4 * 2
        for a, b, c, d in zip(fast[0], slow[0], fast[1], slow[1]):
            assert list(a) == list(b) and np.array_equal(c, d)
    # the array serialiser agrees with the reference-pinned loop codec, clamps included
    big = np.arange(35 * 40).reshape(35, 40) % 10
    toks, pos = D.encode_example_np(big, big[:3, :5])
    want = D.encode_example(big.tolist(), big[:3, :5].tolist())
    assert toks.tolist() == want and np.array_equal(pos, D.compute_positions_3d(want))


def test_seeded_weight_generators_share_one_stream():
    """The product's seeded random-init weights (benchmark, sharded runs) and the oracle's
    (parity tests, golden fixtures) come from the same generator stream: tensor for tensor equal."""
    import torch
    from mdlarc_scale_b200 import synthetic
    from oracle import arc_model as om
    for size, seed, gain in (("tiny", 0, 1.0), ("tiny", 3, 8.0), ("small", 0, 8.0)):
        cfg_d, mine = synthetic.seeded_weights(size, seed, gain)
        cfg = om.make_config(size, max_seq_len=cfg_d["max_seq_len"])
        theirs = om.round_bf16(om.init_state(cfg, seed=seed, embed_gain=gain))
        assert set(mine) == set(theirs)
        for k in mine:
            assert torch.equal(mine[k], theirs[k]), (size, seed, k)
        for f in ("d_model", "n_heads", "n_layers", "d_ff", "vocab_size", "num_examples", "max_x", "max_y", "max_z"):
            assert cfg_d[f] == getattr(cfg, f)


def test_cache_row_pitch_is_the_next_value_16_mod_32():
    """The cache's rows per (sequence, head) are an odd multiple of 16 rows (2 KB): never a multiple of
    64 KB, which is what measurably slows decode attention's streams down."""
    from mdlarc_scale_b200.engine import cache_row_pitch
    for t in list(range(1, 200)) + [1536, 1552, 2048, 2979, 11178]:
        p = cache_row_pitch(t)
        assert t <= p < t + 32 and p % 32 == 16 and cache_row_pitch(p) == p
        assert (p * 128) % 65536 != 0
    assert cache_row_pitch(1536) == 1552 and cache_row_pitch(2048) == 2064
