"""Dataset evaluation and submission writing on the B200 path: the callers either side of
generation + voting, with the reference's signatures and result dictionaries
(``evaluate_task`` src/eval.py:366-509, ``evaluate_dataset`` 512-702, ``generate_submission``
705-878).

Two ways of spreading the work over ranks, behind the same ``rank`` / ``world_size`` arguments:

* ``shard="tasks"`` (default) the reference's partition, ``all_task_ids[rank::world_size]``
  (src/eval.py:569-571): each rank runs whole tasks through ``predict_with_augmentations``,
  i.e. chunks of 16 left-padded prompts, the reference's exact candidate path.
* ``shard="variants"`` (opt-in, the fast path) every (task x test x dihedral x permutation x sample) variant is
  one sequence of one large batch: variants are dealt to ranks by length, prompts are built and
  candidates canonicalised on the device, one all-gather, every rank tallies.  Each rank then
  REPORTS only ``all_task_ids[rank::world_size]``, so a caller that sums the per-rank counters
  (src/eval.py:1203-1208) gets the same totals.  Prompts are not padded here, which is what the
  reference computes for the longest prompts of each of its chunks; for shorter rows the reference
  reads the first token's logits at a padded index (src/inference.py:420-423) and can differ; the
  ``max_seq_len`` clamp is applied per wave of ``wave_size`` rows rather than per chunk of 16.
  Because of those two differences it is not the default of the drop-in entry points.

Seeded vote tie-breaks (``vote_seed``) use the task's position in ``sorted(challenges)`` on both
paths, so a task votes the same way whichever path handled it.

Test-time adaptation needs autograd through the model and stays on the reference module:
``tta_steps > 0`` raises ``NotImplementedError``.
"""
from __future__ import annotations

import json
import random
from pathlib import Path

import numpy as np
import torch

from . import fanout, sharding
from .inference import _resolve_engine, augmented_constraints, predict_with_augmentations
from .voting import aaivr_predict, compute_voting_stats


def grids_equal(grid1, grid2) -> bool:
    """src/eval.py:93-100 (rows compared pairwise after a length check)."""
    if len(grid1) != len(grid2):
        return False
    return all(r1 == r2 for r1, r2 in zip(grid1, grid2, strict=True))


def _no_tta(tta_steps: int) -> None:
    if tta_steps and tta_steps > 0:
        raise NotImplementedError("test-time adaptation needs autograd; run it on the reference module "
                                  "(src/eval.py:144-363) and evaluate the adapted weights here")


def _score_task(task_id: str, task: dict, tops: list, stats: list, solutions) -> dict:
    """Per-task result dictionary of evaluate_task (src/eval.py:418-509) from its votes."""
    res = {"task_id": task_id, "test_outputs": [], "correct_at_1": [], "correct_at_2": [], "voting_stats": []}
    for test_idx in range(len(task["test"])):
        top = tops[test_idx]
        res["voting_stats"].append(stats[test_idx])
        res["test_outputs"].append(top)
        if solutions is not None and test_idx < len(solutions):
            truth = solutions[test_idx]
            res["correct_at_1"].append(len(top) > 0 and grids_equal(top[0], truth))
            res["correct_at_2"].append(any(grids_equal(p, truth) for p in top[:2]))
        else:
            res["correct_at_1"].append(None)
            res["correct_at_2"].append(None)
    v1 = [c for c in res["correct_at_1"] if c is not None]
    v2 = [c for c in res["correct_at_2"] if c is not None]
    res["pass_at_1"] = all(v1) if v1 else None
    res["pass_at_2"] = all(v2) if v2 else None
    res["fractional_at_1"] = sum(v1) / len(v1) if (len(v1) == len(res["correct_at_1"]) and v1) else None
    res["fractional_at_2"] = sum(v2) / len(v2) if (len(v2) == len(res["correct_at_2"]) and v2) else None
    return res


def _vote_rng(vote_seed, task_index: int, test_idx: int):
    """None keeps the reference's unseeded tie-breaks (src/eval.py:468); a seed makes them reproducible."""
    return None if vote_seed is None else random.Random(vote_seed + 1000003 * task_index + test_idx)


def evaluate_task(model, task: dict, task_id: str, device, example_id_map: dict | None = None,
                  use_train_examples: bool = True, solutions=None, num_color_perms: int = 8, top_k: int = 2,
                  max_output_tokens: int = 900, num_samples: int = 1, sample_temperature: float = 0.0,
                  sample_top_k: int | None = None, constrain_decoding: bool = False,
                  palette_penalty: float = 2.0, shape_penalty: float = 2.0, tta_steps: int = 0,
                  tta_lr: float = 0.0, tta_weight_decay: float = 0.0, *, vote_seed: int | None = None,
                  task_index: int = 0) -> dict:
    _no_tta(tta_steps)
    example_id = example_id_map.get(task_id) if example_id_map else 0
    if example_id is None:
        example_id = 0
    tops, stats = [], []
    for test_idx in range(len(task["test"])):
        test_input = task["test"][test_idx]["input"]
        preds = predict_with_augmentations(
            model, task, test_idx, device, example_id=example_id, use_train_examples=use_train_examples,
            num_color_perms=num_color_perms, max_output_tokens=max_output_tokens, num_samples=num_samples,
            sample_temperature=sample_temperature, sample_top_k=sample_top_k,
            constrain_decoding=constrain_decoding, palette_penalty=palette_penalty, shape_penalty=shape_penalty)
        stats.append(compute_voting_stats(preds, test_input=test_input))
        tops.append(aaivr_predict(preds, top_k=top_k, test_input=test_input,
                                  rng=_vote_rng(vote_seed, task_index, test_idx)))
    return _score_task(task_id, task, tops, stats, solutions)


def _variant_constraints(tasks, table, vt, palette_penalty, shape_penalty) -> dict:
    """Per-variant palette masks and target shapes (src/inference.py:798-808, 842-875)."""
    n = len(vt)
    mask = np.ones((n, 10), np.uint8)
    shape = np.full((n, 2), -1, np.int32)
    bounds = np.flatnonzero(np.diff(vt.template, prepend=-1, append=-1))
    for b0, b1 in zip(bounds[:-1].tolist(), bounds[1:].tolist()):
        info = [(int(vt.dihedral[i]), table.perm_tuple(int(vt.perm[i]))) for i in range(b0, b1)]
        palettes, shapes = augmented_constraints(tasks[int(vt.task[b0])], int(vt.test_idx[b0]), info)
        for k, (pal, shp) in enumerate(zip(palettes, shapes)):
            if pal:
                mask[b0 + k] = 0
                for c in pal:
                    if 0 <= c < 10:
                        mask[b0 + k, c] = 1
            if shp is not None:
                shape[b0 + k] = shp
    return dict(palette_mask=mask, target_shape=shape, palette_penalty=float(palette_penalty),
                shape_penalty=float(shape_penalty), disallow_tokens=(10, 12))


def predict_all_variants(model, tasks: list[dict], device, example_ids: list[int], use_train_examples=True,
                         num_color_perms=8, top_k=2, max_output_tokens=900, num_samples=1,
                         sample_temperature=0.0, sample_top_k=None, constrain_decoding=False,
                         palette_penalty=2.0, shape_penalty=2.0, rank=0, world_size=1, vote_seed=None,
                         group=None, wave_size: int = 1024, vote_task_index: list[int] | None = None):
    """Votes and voting statistics of every (task, test input), computed cooperatively by all ranks.

    Returns ``(tops, stats)``: dicts keyed by ``(task_index, test_idx)``, identical on every rank when
    ``vote_seed`` is given (unseeded tie-breaks may order equal counts differently per rank).
    ``vote_task_index[i]`` is the number that seeds task ``i``'s tie-break rng (default ``i``).
    """
    engine = _resolve_engine(model, device)
    table = fanout.TaskTable(tasks, engine.device, num_color_perms=num_color_perms,
                             use_train_examples=use_train_examples)
    vt = table.variants(num_samples)
    cons = _variant_constraints(tasks, table, vt, palette_penalty, shape_penalty) if constrain_decoding else None
    ex = np.asarray(example_ids, np.int32)[vt.task] if engine.use_example_embedding else None
    seed = 0
    if sample_temperature > 0:
        seed = int(torch.randint(0, 2 ** 62, (1,)).item())   # torch.manual_seed makes sampling reproducible
        if world_size > 1:
            import torch.distributed as dist
            t = torch.tensor([seed], dtype=torch.int64, device=engine.device)
            dist.broadcast(t, src=0, group=group)
            seed = int(t.item())
    records = sharding.generate_sharded_records(
        table, vt, int(max_output_tokens), rank, world_size, engine, group=group, wave_size=wave_size,
        example_ids=ex, constraints=cons, temperature=float(sample_temperature), top_k=int(sample_top_k or 0),
        sample_seed=seed, max_seq_len=engine.max_seq_len)
    tallies = fanout.tally_records(records, vt)
    tops, stats = {}, {}
    for key, (ranked_fn, n_total, n_valid) in tallies.items():
        seed_index = key[0] if vote_task_index is None else int(vote_task_index[key[0]])
        votes = ranked_fn(_vote_rng(vote_seed, seed_index, key[1]) or random.Random())
        tops[key] = [g for g, _ in votes[:top_k]]
        counts = [c for _, c in ranked_fn(random.Random(0))]
        top = counts[0] if counts else 0
        stats[key] = {"total_predictions": n_total, "valid_predictions": n_valid,
                      "invalid_predictions": n_total - n_valid, "unique_grids": len(counts),
                      "top_vote_count": top, "vote_distribution": counts[:10],
                      "confidence": (top / n_valid) if (counts and n_valid > 0) else 0.0}
    return tops, stats


def _example_id(example_id_map, task_id) -> int:
    e = example_id_map.get(task_id) if example_id_map else 0
    return 0 if e is None else int(e)


def _variant_votes(model, challenges, task_ids, device, example_id_map, rank, world_size, vote_seed, group,
                   wave_size, **gen):
    """(tops, stats) per task id via the variant-sharded path; ids of tasks it cannot represent.
    ``task_ids`` must be in the caller's canonical (sorted) order: a task's position in it seeds its
    tie-break rng, the same number the per-task path uses."""
    good, bad = [], []
    for tid in task_ids:
        try:
            fanout.TaskTable([challenges[tid]], "cpu", num_color_perms=1,
                             use_train_examples=gen.get("use_train_examples", True))
            good.append(tid)
        except ValueError:
            bad.append(tid)
    out = {}
    if good:
        tasks = [challenges[t] for t in good]
        tops, stats = predict_all_variants(model, tasks, device, [_example_id(example_id_map, t) for t in good],
                                           rank=rank, world_size=world_size, vote_seed=vote_seed, group=group,
                                           wave_size=wave_size,
                                           vote_task_index=[task_ids.index(t) for t in good], **gen)
        for ti, tid in enumerate(good):
            n_tests = len(challenges[tid]["test"])
            out[tid] = ([tops[(ti, k)] for k in range(n_tests)], [stats[(ti, k)] for k in range(n_tests)])
    return out, bad


def evaluate_dataset(model, challenges: dict, device, example_id_map: dict | None = None,
                     use_train_examples: bool = True, solutions: dict | None = None, num_color_perms: int = 8,
                     top_k: int = 2, max_output_tokens: int = 900, num_samples: int = 1,
                     sample_temperature: float = 0.0, sample_top_k: int | None = None,
                     constrain_decoding: bool = False, palette_penalty: float = 2.0, shape_penalty: float = 2.0,
                     tta_steps: int = 0, tta_lr: float = 0.0, tta_weight_decay: float = 0.0,
                     tta_batch_tasks: int = 1, show_progress: bool = True, rank: int = 0, world_size: int = 1,
                     *, shard: str = "tasks", vote_seed: int | None = None, group=None,
                     wave_size: int = 1024) -> dict:
    """Same arguments, partition of REPORTED tasks and result dictionary as src/eval.py:512-702."""
    _no_tta(tta_steps)
    if shard not in ("variants", "tasks"):
        raise ValueError("shard must be 'variants' or 'tasks'")
    all_task_ids = sorted(challenges.keys())
    my_task_ids = all_task_ids[rank::world_size]
    gen = dict(use_train_examples=use_train_examples, num_color_perms=num_color_perms, top_k=top_k,
               max_output_tokens=max_output_tokens, num_samples=num_samples,
               sample_temperature=sample_temperature, sample_top_k=sample_top_k,
               constrain_decoding=constrain_decoding, palette_penalty=palette_penalty, shape_penalty=shape_penalty)
    voted, per_task_path = {}, set(my_task_ids)
    if shard == "variants":
        voted, bad = _variant_votes(model, challenges, all_task_ids, device, example_id_map, rank, world_size,
                                    vote_seed, group, wave_size, **gen)
        per_task_path = set(bad) & set(my_task_ids)
    results = {"total_tasks": len(challenges), "my_tasks": len(my_task_ids), "correct_at_1": 0, "correct_at_2": 0,
               "total_test_examples": 0, "arc_score_at_1": 0.0, "arc_score_at_2": 0.0, "arc_tasks_scored": 0,
               "per_task_results": {}}
    for task_id in my_task_ids:
        task = challenges[task_id]
        sol = solutions.get(task_id) if solutions else None
        if task_id in per_task_path:
            tr = evaluate_task(model, task, task_id, device, example_id_map=example_id_map, solutions=sol,
                               vote_seed=vote_seed, task_index=all_task_ids.index(task_id), **gen)
        else:
            tr = _score_task(task_id, task, voted[task_id][0], voted[task_id][1], sol)
        results["per_task_results"][task_id] = tr
        results["total_test_examples"] += len(task["test"])
        if tr["pass_at_1"] is True:
            results["correct_at_1"] += 1
        if tr["pass_at_2"] is True:
            results["correct_at_2"] += 1
        if tr["fractional_at_1"] is not None and tr["fractional_at_2"] is not None:
            results["arc_score_at_1"] += tr["fractional_at_1"]
            results["arc_score_at_2"] += tr["fractional_at_2"]
            results["arc_tasks_scored"] += 1
    my_total = len(my_task_ids)
    results["accuracy_at_1"] = results["correct_at_1"] / my_total if my_total > 0 else 0.0
    results["accuracy_at_2"] = results["correct_at_2"] / my_total if my_total > 0 else 0.0
    if results["arc_tasks_scored"] > 0:
        results["arc_score_at_1"] /= results["arc_tasks_scored"]
        results["arc_score_at_2"] /= results["arc_tasks_scored"]
    else:
        results["arc_score_at_1"] = results["arc_score_at_2"] = None
    return results


def generate_submission(model, challenges: dict, output_path, device, example_id_map: dict | None = None,
                        use_train_examples: bool = True, num_color_perms: int = 8, top_k: int = 2,
                        max_output_tokens: int = 900, num_samples: int = 1, sample_temperature: float = 0.0,
                        sample_top_k: int | None = None, constrain_decoding: bool = False,
                        palette_penalty: float = 2.0, shape_penalty: float = 2.0, tta_steps: int = 0,
                        tta_lr: float = 0.0, tta_weight_decay: float = 0.0, tta_batch_tasks: int = 1,
                        show_progress: bool = True, *, shard: str = "tasks", vote_seed: int | None = None,
                        rank: int = 0, world_size: int = 1, group=None, wave_size: int = 1024) -> dict:
    """Write the submission file of src/eval.py:705-878: ``{task_id: [{"attempt_1": grid,
    "attempt_2": grid}, ...]}`` in the order of ``challenges``, ``[[0]]`` when nothing was voted, the
    first attempt repeated when there is no second.  With ``world_size > 1`` (variant sharding)
    every rank computes the same votes when ``vote_seed`` is given and rank 0 writes the file.
    Returns the submission dictionary."""
    _no_tta(tta_steps)
    gen = dict(use_train_examples=use_train_examples, num_color_perms=num_color_perms, top_k=min(top_k, 2),
               max_output_tokens=max_output_tokens, num_samples=num_samples,
               sample_temperature=sample_temperature, sample_top_k=sample_top_k,
               constrain_decoding=constrain_decoding, palette_penalty=palette_penalty, shape_penalty=shape_penalty)
    task_ids = list(challenges.keys())
    sorted_ids = sorted(task_ids)      # a task's position here seeds its tie-break rng, as in evaluate_dataset
    voted, bad = {}, task_ids
    if shard == "variants":
        voted, bad = _variant_votes(model, challenges, sorted_ids, device, example_id_map, rank, world_size,
                                    vote_seed, group, wave_size, **gen)
    elif shard != "tasks":
        raise ValueError("shard must be 'variants' or 'tasks'")
    for task_id in bad:
        tr = evaluate_task(model, challenges[task_id], task_id, device, example_id_map=example_id_map,
                           vote_seed=vote_seed, task_index=sorted_ids.index(task_id), **gen)
        voted[task_id] = (tr["test_outputs"], tr["voting_stats"])
    submission = {}
    for task_id in task_ids:
        entries = []
        for top in voted[task_id][0]:
            first = top[0] if len(top) > 0 else [[0]]
            entries.append({"attempt_1": first, "attempt_2": top[1] if len(top) > 1 else first})
        submission[task_id] = entries
    if rank == 0:
        output_path = Path(output_path)
        output_path.parent.mkdir(parents=True, exist_ok=True)
        with open(output_path, "w") as f:
            json.dump(submission, f)
    return submission
