"""evaluate_dataset / generate_submission against result dictionaries of the reference's own
functions (tests/golden/eval.json: src/eval.py run on canned candidate lists).  No GPU: candidate
generation is replaced by the same canned lists, and the variant-sharded path by votes computed
from them, so what is checked is scoring, the per-rank partition and the submission format."""
import json

import pytest
import torch

from mdlarc_scale_b200 import data, evaluation, voting
from mdlarc_scale_b200.data import generate_color_permutations


def canned_predictions(task, test_idx, num_color_perms, solution, rng_grid):
    """Same construction as tests/golden/make_golden.py:canned_predictions."""
    perms = generate_color_permutations(num_color_perms, seed=42)
    wrong = [[(c + 1) % 10 for c in row] for row in solution]
    noise = rng_grid
    first, second = (solution, wrong) if test_idx % 2 == 0 else (wrong, solution)
    if len(task["train"]) == 3:
        second = noise
    if len(task["train"]) == 2:
        first, second = wrong, noise
    out = []
    for d in range(8):
        for p in range(num_color_perms):
            perm = tuple(int(v) for v in perms[p]) if p > 0 else None
            k = d * num_color_perms + p
            g = first if k % 8 < 4 else second if k % 8 < 7 else noise
            if k == 5:
                out.append((None, d, perm))
            elif k == 9:
                out.append(([[1, 2], [3]], d, perm))
            elif k == 11:
                out.append(([list(r) for r in task["test"][test_idx]["input"]], 0, None))
            else:
                t = data.DIHEDRAL_TRANSFORMS[d](g)
                if perm is not None:
                    t = [[perm[c] for c in row] for row in t]
                out.append((t, d, perm))
    return out


@pytest.fixture()
def setup(golden_eval, monkeypatch):
    import numpy as np
    from mdlarc_scale_b200 import synthetic
    challenges, solutions = golden_eval["challenges"], golden_eval["solutions"]
    full = golden_eval["solutions_full"]

    def fake_predict(model, task, test_idx, device, **kw):
        tid = next(k for k, v in challenges.items() if v is task)
        rng = np.random.default_rng(1000 * len(task["train"]) + 17 * test_idx + len(full[tid][test_idx]))
        return canned_predictions(task, test_idx, kw["num_color_perms"], full[tid][test_idx],
                                  synthetic.random_grid(rng, 1, 4))

    monkeypatch.setattr(evaluation, "predict_with_augmentations", fake_predict)

    def fake_variant_votes(model, ch, task_ids, device, example_id_map, rank, world, vote_seed, group, wave, **gen):
        out = {}
        for tid in task_ids:
            tops, stats = [], []
            for k in range(len(ch[tid]["test"])):
                preds = fake_predict(None, ch[tid], k, None, num_color_perms=gen["num_color_perms"])
                test_input = ch[tid]["test"][k]["input"]
                tops.append(voting.aaivr_predict(preds, top_k=gen["top_k"], test_input=test_input))
                stats.append(voting.compute_voting_stats(preds, test_input=test_input))
            out[tid] = (tops, stats)
        return out, []

    return challenges, solutions, fake_variant_votes


def _norm(x):
    return json.loads(json.dumps(x))


@pytest.mark.parametrize("shard", ["tasks", "variants"])
def test_evaluate_dataset_matches_reference_results(golden_eval, setup, monkeypatch, shard):
    challenges, solutions, fake_variant_votes = setup
    if shard == "variants":
        monkeypatch.setattr(evaluation, "_variant_votes", fake_variant_votes)
    n = golden_eval["num_color_perms"]
    for key, want in golden_eval["dataset"].items():
        rank, world = (int(v) for v in key.split("/"))
        got = evaluation.evaluate_dataset(None, challenges, torch.device("cpu"), solutions=solutions,
                                          num_color_perms=n, top_k=2, show_progress=False, rank=rank,
                                          world_size=world, shard=shard)
        assert _norm(got) == want, key
    # the counters a caller all-reduces over ranks (src/eval.py:1203-1208) add up to the one-rank run
    one = golden_eval["dataset"]["0/1"]
    for field in ("correct_at_1", "correct_at_2", "total_test_examples", "my_tasks", "arc_tasks_scored"):
        assert sum(golden_eval["dataset"][f"{r}/2"][field] for r in range(2)) == one[field]


@pytest.mark.parametrize("shard", ["tasks", "variants"])
def test_generate_submission_matches_reference_file(golden_eval, setup, monkeypatch, tmp_path, shard):
    challenges, _, fake_variant_votes = setup
    if shard == "variants":
        monkeypatch.setattr(evaluation, "_variant_votes", fake_variant_votes)
    path = tmp_path / "deep" / "submission.json"
    sub = evaluation.generate_submission(None, challenges, path, torch.device("cpu"),
                                         num_color_perms=golden_eval["num_color_perms"], show_progress=False,
                                         shard=shard)
    assert json.loads(path.read_text()) == golden_eval["submission"] == _norm(sub)
    assert list(sub.keys()) == list(challenges.keys())


def test_submission_fallbacks_and_errors(tmp_path, monkeypatch):
    task = {"train": [], "test": [{"input": [[1]]}, {"input": [[2]]}]}
    monkeypatch.setattr(evaluation, "predict_with_augmentations",
                        lambda model, t, k, dev, **kw: [] if k == 0 else [([[5]], 0, None)])
    sub = evaluation.generate_submission(None, {"a": task}, tmp_path / "s.json", "cpu", shard="tasks")
    assert sub == {"a": [{"attempt_1": [[0]], "attempt_2": [[0]]},          # src/eval.py:828-838
                         {"attempt_1": [[5]], "attempt_2": [[5]]}]}
    with pytest.raises(NotImplementedError):
        evaluation.evaluate_dataset(None, {"a": task}, "cpu", tta_steps=3)
    with pytest.raises(ValueError):
        evaluation.evaluate_dataset(None, {"a": task}, "cpu", shard="rows")
    assert evaluation.grids_equal([[1, 2]], [[1, 2]]) and not evaluation.grids_equal([[1, 2]], [[1, 2], [3]])
