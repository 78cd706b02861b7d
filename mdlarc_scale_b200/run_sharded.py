"""Sharded generation + AAIVR vote over synthetic tasks (the medium 400 x 8 x 20 configuration by
default), one process per GPU:

    python -m mdlarc_scale_b200.run_sharded [--size medium --tasks 400 --perms 20 --max-new 931]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P -m mdlarc_scale_b200.run_sharded ...

Every rank decodes its share of the (task x dihedral x colour-permutation) variants into its
slice of one int32 buffer, a single all-gather completes the buffer, and every rank votes.
Rank 0 prints one JSON line with timings and a checksum of the voted grids, which must not depend
on the number of ranks.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import time

import numpy as np
import torch

from . import sharding, synthetic
from .engine import Engine
from .synthetic import seeded_weights


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", default="medium")
    ap.add_argument("--tasks", type=int, default=400)
    ap.add_argument("--perms", type=int, default=20)
    ap.add_argument("--max-new", type=int, default=931)
    ap.add_argument("--hw-max", type=int, default=30)
    ap.add_argument("--wave", type=int, default=1024)
    ap.add_argument("--embed-gain", type=float, default=8.0)
    ap.add_argument("--seed", type=int, default=2)
    ap.add_argument("--evaluate", action="store_true",
                    help="run evaluate_dataset (variant sharding behind rank / world_size) and sum the "
                         "per-rank counters as src/eval.py:1203-1208 does")
    ap.add_argument("--device-fanout", action="store_true",
                    help="build prompts and canonical candidate records with the fan-out kernels")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    cfg, sd = seeded_weights(args.size, 0, args.embed_gain)
    engine = Engine(sd, cfg, dev)
    tasks = synthetic.capped_tasks(args.seed, args.tasks, 2, 4, 1, args.hw_max, 2048)
    if args.evaluate:
        return main_evaluate(args, tasks, engine, rank, world, dev, dist)
    if args.device_fanout:
        return main_device_fanout(args, tasks, engine, rank, world, dev, dist)
    t0 = time.perf_counter()
    variants = sharding.enumerate_variants(tasks, num_color_perms=args.perms)
    t_enum = time.perf_counter() - t0
    torch.cuda.synchronize(dev)
    if dist is not None:
        dist.barrier()
    t1 = time.perf_counter()
    buf = sharding.generate_sharded(variants, args.max_new, rank, world, sharding.engine_wave_fn(engine),
                                    dev, wave_size=args.wave)
    torch.cuda.synchronize(dev)
    t_gen = time.perf_counter() - t1
    t2 = time.perf_counter()
    layout = sharding.gather_layout([len(v.tokens) for v in variants], world)
    cands = sharding.candidates_from_tokens(variants, buf.cpu().numpy(), layout)
    votes = sharding.vote_all(tasks, cands, top_k=2, seed=7)
    t_vote = time.perf_counter() - t2
    digest = hashlib.sha256(json.dumps(sorted((list(k), v) for k, v in votes.items())).encode()).hexdigest()
    if dist is not None:
        t = torch.tensor([t_gen], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_gen = float(t.item())
    if rank == 0:
        # tokens up to and including each row's first END (all of the row if it never ended)
        has_end = (buf == 13).any(dim=1)
        first_end = (buf == 13).int().argmax(dim=1)
        gen_tokens = int(torch.where(has_end, first_end + 1, torch.full_like(first_end, buf.shape[1]))
                         [torch.from_numpy(layout >= 0).to(buf.device)].sum().item())
        print(json.dumps({
            "workload": f"{args.size}: {args.tasks} tasks x 8 dihedral x {args.perms} colour permutations",
            "n_gpus": world, "variants": len(variants), "max_new": args.max_new,
            "enumerate_s": t_enum, "generate_and_gather_s": t_gen, "decode_grids_and_vote_s": t_vote,
            "generated_tokens": gen_tokens, "generated_tokens_per_s": gen_tokens / t_gen,
            "tasks_with_votes": sum(1 for v in votes.values() if v), "votes_sha256": digest}), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main_evaluate(args, tasks, engine, rank, world, dev, dist):
    from . import evaluation
    challenges = {f"task{i:04d}": t for i, t in enumerate(tasks)}
    # stand-in solutions (the synthetic tasks have none): the first train output of each task
    solutions = {tid: [t["train"][0]["output"] for _ in t["test"]] for tid, t in challenges.items()}
    torch.cuda.synchronize(dev)
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    res = evaluation.evaluate_dataset(engine, challenges, dev, solutions=solutions, num_color_perms=args.perms,
                                      top_k=2, max_output_tokens=args.max_new, show_progress=False, rank=rank,
                                      world_size=world, vote_seed=7, wave_size=args.wave, shard="variants")
    torch.cuda.synchronize(dev)
    wall = time.perf_counter() - t0
    fields = ["correct_at_1", "correct_at_2", "total_test_examples", "my_tasks", "arc_tasks_scored"]
    counts = torch.tensor([res[f] for f in fields], dtype=torch.int64, device=dev)
    outputs = {tid: tr["test_outputs"] for tid, tr in res["per_task_results"].items()}
    if dist is not None:
        dist.all_reduce(counts)
        gathered = [None] * world
        dist.all_gather_object(gathered, outputs)
        outputs = {k: v for part in gathered for k, v in part.items()}
    if rank == 0:
        digest = hashlib.sha256(json.dumps(sorted(outputs.items())).encode()).hexdigest()
        print(json.dumps({"workload": f"evaluate_dataset, {args.size}: {args.tasks} tasks x 8 x {args.perms}",
                          "n_gpus": world, "wall_s": wall, **dict(zip(fields, counts.tolist())),
                          "tasks_reported": len(outputs), "outputs_sha256": digest}), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main_device_fanout(args, tasks, engine, rank, world, dev, dist):
    from . import fanout
    t0 = time.perf_counter()
    table = fanout.TaskTable(tasks, dev, num_color_perms=args.perms)
    vt = table.variants()
    t_enum = time.perf_counter() - t0
    torch.cuda.synchronize(dev)
    if dist is not None:
        dist.barrier()
    t1 = time.perf_counter()
    records = sharding.generate_sharded_records(table, vt, args.max_new, rank, world, engine, wave_size=args.wave)
    torch.cuda.synchronize(dev)
    t_gen = time.perf_counter() - t1
    t2 = time.perf_counter()
    votes = fanout.vote_records(records, vt, top_k=2, seed=7)
    t_vote = time.perf_counter() - t2
    digest = hashlib.sha256(json.dumps(sorted((list(k), v) for k, v in votes.items())).encode()).hexdigest()
    if dist is not None:
        t = torch.tensor([t_gen], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_gen = float(t.item())
    if rank == 0:
        gen_tokens = int(fanout.record_fields(records)[4].astype(np.int64).sum())
        print(json.dumps({
            "workload": f"{args.size}: {args.tasks} tasks x 8 dihedral x {args.perms} colour permutations",
            "fanout": "device", "n_gpus": world, "variants": len(vt), "max_new": args.max_new,
            "enumerate_s": t_enum, "generate_and_gather_s": t_gen, "decode_grids_and_vote_s": t_vote,
            "generated_tokens": gen_tokens, "generated_tokens_per_s": gen_tokens / t_gen,
            "tasks_with_votes": sum(1 for v in votes.values() if v), "votes_sha256": digest}), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
