"""Generate the golden fixtures in this directory by running the REFERENCE implementation.

Run where the reference source tree is available (it is imported read-only, never copied):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

Inputs are seeded; weights come from oracle.arc_model.init_state loaded into the reference's
TinyTransformer with ``load_state_dict(strict=True)`` (so names and shapes are checked too).
Outputs: model_tiny.npz (fp32 logits + greedy tokens), tokens.json (codec / position /
augmentation known answers), votes.json (AAIVR results with seeded tie-break rngs), eval.json
(result dictionaries of the reference's evaluate_dataset / generate_submission for canned
candidate lists).  ``--only NAME`` (tokens, votes, model, eval) rewrites one of them.
"""
import json
import random
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
if len(sys.argv) < 2:
    raise SystemExit("usage: make_golden.py /path/to/reference")
REF = sys.argv[1]
sys.path.insert(0, REF)
sys.dont_write_bytecode = True

from src import data as rdata  # noqa: E402  (reference)
from src import inference as rinf  # noqa: E402
from src import transformer as rtr  # noqa: E402
from src import voting as rvote  # noqa: E402

from mdlarc_scale_b200 import synthetic  # noqa: E402
from mdlarc_scale_b200.inference import pad_prompts  # noqa: E402
from oracle import arc_model as om  # noqa: E402

torch.manual_seed(0)
torch.set_num_threads(4)


def reference_model(cfg: om.Config, sd: dict):
    m = rtr.create_tiny_model(max_seq_len=cfg.max_seq_len)
    m.load_state_dict(sd, strict=True)
    return m.eval()


def golden_model():
    cfg = om.make_config("tiny", max_seq_len=4096)
    out = {}
    tasks = synthetic.capped_tasks(11, 3, 2, 3, 1, 7, None)
    prompts, positions = synthetic.prompts_for(tasks)
    for wname, kw in (("plain", {}), ("varied", dict(embed_gain=8.0))):
        sd = om.round_bf16(om.perturb_state(om.init_state(cfg, seed=0, **kw), seed=1))
        out[f"{wname}_weight_abs_sum"] = np.float64(sum(float(v.abs().double().sum()) for v in sd.values()))
        model = reference_model(cfg, sd)
        for pad in ("right", "left"):
            ids, pos, mask = pad_prompts(prompts, positions, left=(pad == "left"))
            ids_t, pos_t, mask_t = torch.from_numpy(ids), torch.from_numpy(pos), torch.from_numpy(mask)
            ex = torch.tensor([3, 0, 7])
            with torch.no_grad():
                logits = model(ids_t, pos_t, ex, mask_t)
                toks = rinf.generate_output(model, ids_t, pos_t, ex, mask_t, max_new_tokens=48)
                toks_nostop = rinf.generate_output(model, ids_t, pos_t, ex, mask_t, max_new_tokens=24,
                                                   stop_on_end=False)
            key = f"{wname}_{pad}"
            out[key + "_ids"] = ids
            out[key + "_pos"] = pos
            out[key + "_mask"] = mask
            out[key + "_ex"] = ex.numpy()
            out[key + "_logits"] = logits.numpy()
            out[key + "_gen"] = toks.numpy()
            out[key + "_gen_nostop"] = toks_nostop.numpy()
        # soft-constrained decoding (palette + target shape + disallowed tokens), right-padded batch
        ids, pos, mask = pad_prompts(prompts, positions, left=False)
        pm = torch.tensor([[1, 1, 0, 0, 1, 0, 0, 0, 0, 1], [1, 0, 1, 1, 0, 0, 1, 0, 0, 0], [1] * 10], dtype=torch.bool)
        ts = torch.tensor([[3, 4], [-1, -1], [2, 2]])
        cons = rinf.DecodingConstraints(palette_mask=pm, target_shape=ts, palette_penalty=1.5, shape_penalty=2.5)
        with torch.no_grad():
            toks_c = rinf.generate_output(model, torch.from_numpy(ids), torch.from_numpy(pos), torch.tensor([3, 0, 7]),
                                          torch.from_numpy(mask), max_new_tokens=32, stop_on_end=False,
                                          constraints=cons)
        out[f"{wname}_constrained_gen"] = toks_c.numpy()
        out[f"{wname}_constrained_palette"] = pm.numpy()
        out[f"{wname}_constrained_shape"] = ts.numpy()
        # no mask, no example ids: plain causal forward
        ids, pos, _ = pad_prompts(prompts[:1], positions[:1], left=False)
        with torch.no_grad():
            out[f"{wname}_nomask_logits"] = model(torch.from_numpy(ids), torch.from_numpy(pos)).numpy()
        out[f"{wname}_nomask_ids"] = ids
        out[f"{wname}_nomask_pos"] = pos
    np.savez_compressed(HERE / "model_tiny.npz", **out)


def golden_tokens():
    rng = np.random.default_rng(3)
    cases = []
    for _ in range(6):
        gi = synthetic.random_grid(rng, 1, 6)
        go = synthetic.random_grid(rng, 1, 6)
        toks = rdata.encode_example(gi, go) + rdata.encode_example(go, None)
        cases.append({
            "input": gi, "output": go, "tokens": toks,
            "positions": rdata.compute_positions_3d(toks).tolist(),
            "dihedral_in": [f(gi) for f in rdata.DIHEDRAL_TRANSFORMS],
            "decoded": rdata.decode_output_grid(toks),
        })
    streams = [[12, 1, 2, 11, 3, 4, 11, 13], [12, 13], [1, 2, 3], [12, 5, 11, 11, 6, 10, 7, 13, 9],
               [12, 1, 2, 11, 3, 11]]
    decoded = [rdata.decode_output_grid(s) for s in streams]
    # grid-state tracker vs positions: feed continuation tokens one by one
    gs_cases = []
    for c in cases[:3]:
        toks = c["tokens"]
        cut = len(toks) // 2
        ids = torch.tensor([toks[:cut]])
        pos = torch.tensor([c["positions"][:cut]])
        x, y, io = rinf._derive_initial_state_from_prompt(ids, pos, None, 30, 29)
        g = rinf.GridStateUpdater(1, torch.device("cpu"))
        g.set_state(x, y, io)
        track = [g.update(torch.tensor([t])).tolist()[0] for t in toks[cut:]]
        gs_cases.append({"tokens": toks, "cut": cut, "init": [int(x), int(y), bool(io)], "track": track})
    long_row = [[1] * 40 for _ in range(35)]  # exceeds the clamps
    long_toks = rdata.encode_example(long_row, None)
    # constrained-decoding host helpers on a synthetic task with a common output shape
    ctask = synthetic.capped_tasks(5, 1, 3, 3, 2, 5, None)[0]
    shape0 = (len(ctask["train"][0]["output"]), len(ctask["train"][0]["output"][0]))
    for pair in ctask["train"][1:]:
        pair["output"] = [row[:shape0[1]] + [0] * max(0, shape0[1] - len(row)) for row in pair["output"][:shape0[0]]]
        while len(pair["output"]) < shape0[0]:
            pair["output"].append([0] * shape0[1])
    base_palette = sorted(rinf._collect_palette(ctask, 0))
    base_shape = rinf._infer_output_shape(ctask)
    perms = rdata.generate_color_permutations(3, seed=42)
    con_rows = []
    for d in range(8):
        for p in range(3):
            pal = sorted({int(perms[p][c]) for c in base_palette}) if p > 0 else base_palette
            shp = rinf._transform_shape(base_shape, d)
            con_rows.append({"dihedral": d, "perm": p, "palette": pal, "shape": list(shp) if shp else None})
    out = {
        "constraint_task": ctask, "constraint_rows": con_rows,
        "cases": cases, "streams": streams, "decoded": decoded, "grid_state": gs_cases,
        "perms20": rdata.generate_color_permutations(20, seed=42).tolist(),
        "perms3_seed7": rdata.generate_color_permutations(3, seed=7).tolist(),
        "long_positions_tail": rdata.compute_positions_3d(long_toks)[-50:].tolist(),
        "long_n": len(long_toks),
    }
    (HERE / "tokens.json").write_text(json.dumps(out))


def golden_votes():
    rng = np.random.default_rng(9)
    perms = rdata.generate_color_permutations(6, seed=42)
    cases = []
    for case in range(8):
        base = [synthetic.random_grid(rng, 1, 4) for _ in range(3)]
        test_input = base[0]
        preds = []
        for _ in range(int(rng.integers(0, 30))):
            kind = rng.random()
            d = int(rng.integers(0, 8))
            p = int(rng.integers(0, 6))
            perm = tuple(int(v) for v in perms[p]) if p > 0 else None
            g = base[int(rng.integers(0, 3))]
            g = rdata.DIHEDRAL_TRANSFORMS[d](g)
            if perm is not None:
                g = [[perm[c] for c in row] for row in g]
            if kind < 0.1:
                preds.append([None, d, perm])
            elif kind < 0.2:
                preds.append([[[1, 2], [3]], d, perm])       # jagged
            elif kind < 0.25:
                preds.append([[], d, perm])                  # empty
            elif kind < 0.3:
                preds.append([[list(r) for r in test_input], 0, None])  # input copy
            else:
                preds.append([g, d, perm])
        tup = [(g, d, tuple(p) if p is not None else None) for g, d, p in preds]
        votes = rvote.aggregate_votes(tup, test_input=test_input, rng=random.Random(case))
        top2 = rvote.aaivr_predict(tup, top_k=2, test_input=test_input, rng=random.Random(case))
        keep = rvote.aaivr_predict(tup, top_k=3, test_input=test_input, discard_input_copies=False,
                                   rng=random.Random(case + 100))
        stats = rvote.compute_voting_stats(tup, test_input=test_input)
        cases.append({"predictions": preds, "test_input": test_input, "seed": case,
                      "votes": [[g, c] for g, c in votes], "top2": top2, "top3_keep_copies": keep, "stats": stats})
    (HERE / "votes.json").write_text(json.dumps({"cases": cases}))


def canned_predictions(task, test_idx, num_color_perms, solution):
    """Candidate list of one test input, in the reference's order, with an unambiguous top two:
    the true output wins for even test indices, a wrong grid for odd ones; noise has fewer votes."""
    perms = rdata.generate_color_permutations(num_color_perms, seed=42)
    rng = np.random.default_rng(1000 * len(task["train"]) + 17 * test_idx + len(solution))
    wrong = [[(c + 1) % 10 for c in row] for row in solution]
    noise = synthetic.random_grid(rng, 1, 4)
    first, second = (solution, wrong) if test_idx % 2 == 0 else (wrong, solution)
    if len(task["train"]) == 3:
        second = noise          # noise outvotes the other attempt
    if len(task["train"]) == 2:
        first, second = wrong, noise   # a task with both attempts wrong
    out = []
    for d in range(8):
        for p in range(num_color_perms):
            perm = tuple(int(v) for v in perms[p]) if p > 0 else None
            k = d * num_color_perms + p
            g = first if k % 8 < 4 else second if k % 8 < 7 else noise
            if k == 5:
                out.append((None, d, perm))
                continue
            if k == 9:
                out.append(([[1, 2], [3]], d, perm))
                continue
            if k == 11:
                out.append(([list(r) for r in task["test"][test_idx]["input"]], 0, None))   # an input copy
                continue
            t = rdata.DIHEDRAL_TRANSFORMS[d](g)
            if perm is not None:
                t = [[perm[c] for c in row] for row in t]
            out.append((t, d, perm))
    return out


def golden_eval():
    import tempfile

    from src import eval as reval
    tasks = synthetic.capped_tasks(21, 5, 1, 3, 2, 5, None)
    challenges, solutions = {}, {}
    rng = np.random.default_rng(5)
    for i, t in enumerate(tasks):
        tid = f"task{(7 * i) % 5:02d}"
        if i == 1:
            t["test"].append({"input": synthetic.random_grid(rng, 2, 4)})
        challenges[tid] = t
        solutions[tid] = [synthetic.random_grid(rng, 2, 4) for _ in t["test"]]
    del solutions["task01"][-1:]          # one task with a missing solution (unscored)
    n_perms = 3

    def fake_predict(model, task, test_idx, device, **kw):
        tid = next(k for k, v in challenges.items() if v is task)
        sol = solutions_full[tid][test_idx]
        return canned_predictions(task, test_idx, kw["num_color_perms"], sol)

    solutions_full = {k: list(v) for k, v in solutions.items()}
    for tid, t in challenges.items():      # canned candidates need a target even where no solution is scored
        while len(solutions_full[tid]) < len(t["test"]):
            solutions_full[tid].append(synthetic.random_grid(rng, 2, 4))
    reval.predict_with_augmentations = fake_predict

    class Dummy(torch.nn.Module):
        config = None

    model = Dummy()
    out = {"challenges": challenges, "solutions": solutions, "solutions_full": solutions_full, "num_color_perms": n_perms,
           "dataset": {}}
    for world in (1, 2):
        for rank in range(world):
            res = reval.evaluate_dataset(model, challenges, torch.device("cpu"), solutions=solutions,
                                         num_color_perms=n_perms, top_k=2, show_progress=False, rank=rank,
                                         world_size=world)
            out["dataset"][f"{rank}/{world}"] = res
    with tempfile.TemporaryDirectory() as tmp:
        path = Path(tmp) / "sub" / "submission.json"
        reval.generate_submission(model, challenges, path, torch.device("cpu"), num_color_perms=n_perms,
                                  show_progress=False)
        out["submission"] = json.loads(path.read_text())
    (HERE / "eval.json").write_text(json.dumps(out))


if __name__ == "__main__":
    only = sys.argv[sys.argv.index("--only") + 1] if "--only" in sys.argv else None
    for name, fn in (("tokens", golden_tokens), ("votes", golden_votes), ("model", golden_model),
                     ("eval", golden_eval)):
        if only in (None, name):
            fn()
    print("golden fixtures written to", HERE)
