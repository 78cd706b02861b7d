"""The CPU oracle against outputs of the reference implementation (tests/golden)."""
import random

import numpy as np
import torch

from conftest import tuple_preds
from oracle import arc_model as om
from oracle import arc_tokens as ot
from oracle import arc_vote as ov


def _weights(name):
    cfg = om.make_config("tiny", max_seq_len=4096)
    kw = dict(embed_gain=8.0) if name == "varied" else {}
    return cfg, om.round_bf16(om.perturb_state(om.init_state(cfg, seed=0, **kw), seed=1))


def test_weight_stream_is_reproducible(golden_model):
    for name in ("plain", "varied"):
        _, sd = _weights(name)
        s = sum(float(v.abs().double().sum()) for v in sd.values())
        assert abs(s - float(golden_model[f"{name}_weight_abs_sum"])) < 1e-6 * s


def test_forward_matches_reference_logits(golden_model):
    for name in ("plain", "varied"):
        cfg, sd = _weights(name)
        for pad in ("right", "left"):
            k = f"{name}_{pad}"
            mask = torch.from_numpy(golden_model[k + "_mask"])
            got = om.forward(sd, cfg, torch.from_numpy(golden_model[k + "_ids"]),
                             torch.from_numpy(golden_model[k + "_pos"]),
                             torch.from_numpy(golden_model[k + "_ex"]), mask)
            want = torch.from_numpy(golden_model[k + "_logits"])
            # fp32 round-off only; compared on valid positions (padded queries of a left-padded row
            # see no key at all and are backend-defined)
            assert torch.allclose(got[mask], want[mask], atol=2e-5, rtol=1e-5)
        got = om.forward(sd, cfg, torch.from_numpy(golden_model[f"{name}_nomask_ids"]),
                         torch.from_numpy(golden_model[f"{name}_nomask_pos"]))
        assert torch.allclose(got, torch.from_numpy(golden_model[f"{name}_nomask_logits"]), atol=2e-5, rtol=1e-5)


def test_generate_matches_reference_tokens(golden_model):
    for name in ("plain", "varied"):
        cfg, sd = _weights(name)
        for pad in ("right", "left"):
            k = f"{name}_{pad}"
            args = (torch.from_numpy(golden_model[k + "_ids"]), torch.from_numpy(golden_model[k + "_pos"]),
                    torch.from_numpy(golden_model[k + "_ex"]), torch.from_numpy(golden_model[k + "_mask"]))
            got = om.generate(sd, cfg, *args, max_new_tokens=48).tokens.numpy()
            assert np.array_equal(got, golden_model[k + "_gen"]), k
            got = om.generate(sd, cfg, *args, max_new_tokens=24, stop_on_end=False).tokens.numpy()
            assert np.array_equal(got, golden_model[k + "_gen_nostop"]), k


def test_varied_weights_reach_end_and_stay_ragged(golden_model):
    gen = golden_model["varied_right_gen"]
    s = golden_model["varied_right_ids"].shape[1]
    ends = [(row[s:] == 13).any() for row in gen]
    assert any(ends) and not all(ends)


def test_prefill_plus_decode_equals_full_forward(golden_model):
    cfg, sd = _weights("varied")
    k = "varied_right"
    ids, pos = torch.from_numpy(golden_model[k + "_ids"])[:1], torch.from_numpy(golden_model[k + "_pos"])[:1]
    n = int(golden_model[k + "_mask"][0].sum())
    ids, pos = ids[:, :n], pos[:, :n]
    ex = torch.tensor([3])
    r = om.generate(sd, cfg, ids, pos, ex, None, max_new_tokens=6, stop_on_end=False, keep_logits=True)
    full_tokens = r.tokens[0].tolist()
    full_pos = torch.from_numpy(ot.positions_3d(full_tokens))[None]
    logits = om.forward(sd, cfg, r.tokens, full_pos, ex)
    for i, lg in enumerate(r.logits):
        assert torch.allclose(lg[0], logits[0, n - 1 + i], atol=3e-5)


def test_token_codec_positions_dihedral(golden_tokens):
    for c in golden_tokens["cases"]:
        toks = ot.encode_example(c["input"], c["output"]) + ot.encode_example(c["output"], None)
        assert toks == c["tokens"]
        assert ot.positions_3d(toks).tolist() == c["positions"]
        assert [ot.dihedral(c["input"], i) for i in range(8)] == c["dihedral_in"]
        assert ot.decode_output_grid(toks) == c["decoded"]
    for s, d in zip(golden_tokens["streams"], golden_tokens["decoded"]):
        assert ot.decode_output_grid(s) == d
    assert ot.color_permutations(20, 42).tolist() == golden_tokens["perms20"]
    assert ot.color_permutations(3, 7).tolist() == golden_tokens["perms3_seed7"]


def test_grid_state(golden_tokens):
    for c in golden_tokens["grid_state"]:
        toks, cut = c["tokens"], c["cut"]
        pos = ot.positions_3d(toks)
        x, y, io = ot.initial_state(toks[cut - 1], pos[cut - 1], True)
        assert [x, y, io] == c["init"]
        g = ot.GridState(x, y, io)
        assert [list(g.update(t)) for t in toks[cut:]] == c["track"]
        # and the tracker reproduces compute_positions_3d on the true continuation
        assert c["track"] == pos[cut:].tolist()


def test_votes(golden_votes):
    for c in golden_votes["cases"]:
        preds = tuple_preds(c["predictions"])
        votes = ov.aggregate_votes(preds, test_input=c["test_input"], rng=random.Random(c["seed"]))
        assert [[g, n] for g, n in votes] == c["votes"]
        assert ov.aaivr_predict(preds, 2, c["test_input"], rng=random.Random(c["seed"])) == c["top2"]
        assert ov.aaivr_predict(preds, 3, c["test_input"], False, random.Random(c["seed"] + 100)) == c["top3_keep_copies"]


def test_constrained_generate_matches_reference(golden_model):
    for name in ("plain", "varied"):
        cfg, sd = _weights(name)
        k = f"{name}_right"
        cons = dict(palette_mask=torch.from_numpy(golden_model[f"{name}_constrained_palette"]),
                    target_shape=torch.from_numpy(golden_model[f"{name}_constrained_shape"]),
                    palette_penalty=1.5, shape_penalty=2.5, disallow_tokens=(10, 12))
        got = om.generate(sd, cfg, torch.from_numpy(golden_model[k + "_ids"]), torch.from_numpy(golden_model[k + "_pos"]),
                          torch.from_numpy(golden_model[k + "_ex"]), torch.from_numpy(golden_model[k + "_mask"]),
                          max_new_tokens=32, stop_on_end=False, constraints=cons).tokens.numpy()
        assert np.array_equal(got, golden_model[f"{name}_constrained_gen"])
        # the constraints really bite: the unconstrained continuation differs
        S = golden_model[k + "_ids"].shape[1]
        assert not np.array_equal(got[:, S:S + 24], golden_model[k + "_gen_nostop"][:, S:S + 24])
