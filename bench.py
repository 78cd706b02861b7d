#!/usr/bin/env python
"""Benchmark of the hot path: batched greedy generation of the large TinyTransformer, bf16.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the decode-bound large configuration): `--batch` sequences per GPU per step with short
prompts (2 train pairs + test input, grids 3..10 x 3..10), END suppressed, every sequence decoded
for the full 931-token budget over a static KV cache of 1536 positions.  One step = one pass of
the hot path over one such batch: packed prefill + 930 graph-replayed decode steps.  Under
torchrun every rank runs its own batch (weak scaling, no data-path collective).

Prints ONE JSON line (rank 0): generated tokens/s over all GPUs, device-timed (`value`, inputs
resident in HBM) and end to end through `generate_output` from pinned host tensors (`e2e`),
plus the roofline of the dominant kernel (decode attention, HBM-bound), the CPU baseline, clocks.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

MAX_NEW = 931
MAX_NEW_FULL = 931   # the configurations' budget (MAX_NEW may be lowered for profiling runs)
KV_POSITIONS = 1536
MODEL_SIZE = "large"
# DRAM traffic of the decode-attention kernel relative to its algorithmic bytes, measured with one
# ncu capture of the standalone kernel on 256 sequences x 1000 cached positions (1311.5 MB read +
# 4.0 MB written per launch for 1310.72 MB algorithmic); traffic grows in proportion to the cached
# positions, so a full-size launch is scaled by its algorithmic bytes.
ATTN_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.0037
LINEAR_FLOP_PER_TOKEN = 469.9e6          # large model: 2 x matmul parameters


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def measured_tensor_peaks():
    """(burst, sustained) dense bf16 TFLOP/s and whether they are this pool's measured figures."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self._stop = threading.Event()
        self._t = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                parts = [x.strip() for x in out.stdout.strip().split(",")]
                if len(parts) >= 7:
                    self.rows.append(parts)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(float(r[0]) for r in self.rows)
        reasons = []
        for i, name in enumerate(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")):
            if any(r[3 + i].lower().startswith("active") for r in self.rows):
                reasons.append(name)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(self.rows[0][1]), "reasons": reasons,
                "samples": len(self.rows)}


def make_batch(seed: int, n: int):
    from mdlarc_scale_b200 import synthetic
    from mdlarc_scale_b200.inference import pad_prompts
    tasks = synthetic.capped_tasks(seed, n, 2, 2, 3, 10, None)
    prompts, positions = synthetic.prompts_for(tasks)
    return pad_prompts(prompts, positions, left=False)


def model_state():
    """Seeded random-init weights of the large model (reference distributions), rounded to bf16."""
    from mdlarc_scale_b200.synthetic import seeded_weights
    return seeded_weights(MODEL_SIZE, seed=0)


# ---------------------------------------------------------------------------
# CPU baseline / reference arm: the reference project's own generate_output (its files copied to
# oracle/_ref by oracle/make_ref.py) on the host cores; the oracle port only when they are absent
# ---------------------------------------------------------------------------
_REF_MODEL = None


def _reference_model():
    """The reference TinyTransformer (large) holding this benchmark's seeded weights, or None."""
    global _REF_MODEL
    if _REF_MODEL is None:
        from oracle import make_ref  # the timed CPU baseline IS the reference / its port
        if not make_ref.available():
            _REF_MODEL = False
        else:
            mods = make_ref.load_reference_modules("arcref")
            cfg_d, sd = model_state()
            model = mods["transformer"].create_large_model(max_seq_len=cfg_d["max_seq_len"])
            model.load_state_dict(sd, strict=True)
            model.eval()
            _REF_MODEL = (model, mods["inference"].generate_output)
    return _REF_MODEL or None


def cpu_generate_sample(n_seqs: int, n_steps: int, seed: int):
    """Prefill + n_steps greedy tokens of n_seqs sequences of the benchmark's generator on the host
    cores, fp32.  Returns (tokens/s, seconds, kind, mean cached length over the decode steps)."""
    ids, pos, mask = make_batch(seed, n_seqs)
    ids_t, pos_t, mask_t = torch.from_numpy(ids), torch.from_numpy(pos), torch.from_numpy(mask)
    ref = _reference_model()
    t0 = time.perf_counter()
    if ref is not None:
        model, generate_output = ref
        with torch.no_grad():
            out = generate_output(model, ids_t, pos_t, None, mask_t, max_new_tokens=n_steps, stop_on_end=False)
        gen = out.shape[1] - ids.shape[1]
        kind = "reference"
    else:
        from oracle import arc_model as om
        cfg_d, sd = model_state()
        r = om.generate(sd, om.Config(**cfg_d), ids_t, pos_t, None, mask_t, max_new_tokens=n_steps,
                        stop_on_end=False)
        gen = r.tokens.shape[1] - ids.shape[1]
        kind = "port"
    dt = time.perf_counter() - t0
    mean_cache = float(mask.sum(axis=1).mean()) + gen / 2.0
    return n_seqs * gen / dt, dt, kind, mean_cache


def _cpu_sample_text(n_seqs, n_steps, kind, mean_cache, dt=None):
    what = ("the reference's own generate_output (src/inference.py), unmodified" if kind == "reference"
            else "oracle port of generate_output")
    txt = (f"{n_seqs} sequences of the same generator x (prefill + {n_steps} greedy tokens), fp32, {what}; "
           f"mean cached length {mean_cache:.0f} positions (the GPU arm: 1024 sequences x {MAX_NEW} tokens at "
           f"mean cached length ~{252 + MAX_NEW // 2})")
    return txt + (f"; {dt:.1f} s wall" if dt is not None else "")


def run_reference(args, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    n_seqs, n_steps = args.cpu_seqs, args.cpu_steps
    for i in range(args.warmup):
        cpu_generate_sample(2, 4, 1000 + i)
    vals, times, kind, mean_cache = [], [], "port", 0.0
    for i in range(args.steps):
        v, dt, kind, mean_cache = cpu_generate_sample(n_seqs, n_steps, 2000 + i)
        vals.append(v)
        times.append(dt)
    value = float(np.mean(vals))
    line = {
        "impl": "reference", "metric": "generated tokens/s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1000 * float(np.mean(times)), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "cfg4-large-decode", "model": MODEL_SIZE, "sequences_per_gpu_per_step": args.batch,
                   "new_tokens": MAX_NEW, "kv_positions": KV_POSITIONS, "stop_on_end": False,
                   "note": "CPU arm: each step is a bounded sample of this workload (see cpu_baseline.sample)"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": kind,
                         "sample": _cpu_sample_text(n_seqs, n_steps, kind, mean_cache)},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def attention_roofline(engine, session, lens0: np.ndarray, n_layers_sampled: int = 2):
    """Replays the decode-attention kernel on the live KV cache at five points of the decode
    trajectory (same launch shape as inside the graph) and times each launch with CUDA events."""
    import ctypes as C
    from mdlarc_scale_b200 import _lib
    lib = engine.lib
    B, H, T = session.n_seqs, engine.n_heads, session.t_max
    dev = engine.device
    q = torch.randn(B, H, 64, device=dev).to(torch.float16)
    out = torch.empty_like(q)
    layer_bytes = 2 * B * engine.d_model * T * 2
    times, bytes_ = [], []
    for frac in (0.05, 0.25, 0.5, 0.75, 1.0):
        lens = torch.from_numpy((lens0 + int(frac * (MAX_NEW - 1))).astype(np.int32)).to(dev)
        algo = int(lens.sum().item()) * H * 64 * 2 * 2  # K and V rows, bf16, each read once
        for layer in range(n_layers_sampled):
            kptr = session.kv_cache.data_ptr() + layer * layer_bytes
            vptr = kptr + layer_bytes // 2
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _lib.check(lib.arcb_op_decode_attention(q.data_ptr(), kptr, vptr, out.data_ptr(), None, lens.data_ptr(),
                                                    None, B, H, T, 1, None, _lib.ACT_F16,
                                                    torch.cuda.current_stream(dev).cuda_stream))
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1) / 1e3)
            bytes_.append(algo)
    # achieved = sum of bytes / sum of time, so achieved x ms_per_launch = algorithmic_bytes_per_launch
    gbs = float(np.sum(bytes_) / np.sum(times) / 1e9)
    return gbs, float(np.mean(times) * 1e3), float(np.mean(bytes_))


def profile_attention(args):
    """Standalone decode-attention launches of known size (for an ncu capture, or an A/B of the kernel
    variants through their environment switches): `--batch` sequences, 20 heads, `--profile-attn` cached
    positions per sequence, or lengths drawn uniformly from T - spread .. T + spread with
    `--profile-attn-spread`; prints the algorithmic bytes and the CUDA-event time of every launch."""
    from mdlarc_scale_b200 import _lib
    lib = _lib.load()
    B, H, T = args.batch, 20, args.profile_attn
    spread = max(0, min(args.profile_attn_spread, T - 1))
    t_max = max(T + spread, args.profile_attn_pitch)   # rows between two (sequence, head) streams of the cache
    dev = torch.device("cuda", 0)
    q = torch.randn(B, H, 64, device=dev).to(torch.float16)
    kv = torch.empty(2, B, H, t_max, 64, device=dev, dtype=torch.bfloat16)
    kv.view(torch.int16).random_(0, 16128)   # bit patterns of finite non-negative bf16 values below 0.5
    out = torch.empty_like(q)
    lens_np = np.random.default_rng(3).integers(T - spread, T + spread + 1, size=B).astype(np.int32)
    lens = torch.from_numpy(lens_np).to(dev)
    ms = []
    for _ in range(8 if spread or B > 256 else 4):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        _lib.check(lib.arcb_op_decode_attention(q.data_ptr(), kv[0].data_ptr(), kv[1].data_ptr(), out.data_ptr(), None,
                                                lens.data_ptr(), None, B, H, t_max, 1, None, _lib.ACT_F16,
                                                torch.cuda.current_stream(dev).cuda_stream))
        e1.record()
        e1.synchronize()
        ms.append(e0.elapsed_time(e1))
    algo = int(lens_np.sum()) * H * 64 * 2 * 2
    warm = sorted(ms[2:])
    print(json.dumps({"profile": "decode attention", "batch": B, "heads": H, "cached_positions": T, "spread": spread, "capacity": t_max,
                      "algorithmic_bytes_per_launch": algo, "ms_per_launch": ms,
                      "gbs_last": algo / ms[-1] / 1e6, "gbs_median": algo / warm[len(warm) // 2] / 1e6}))


def profile_prefill(args):
    """Prefill-only pass of the prefill-heavy large configuration: prompts of `--profile-prefill`
    train pairs of 30x30 grids plus a 30x30 test input (5 pairs = 10 247 tokens), about 64k packed
    tokens per call; prints prompt tokens/s and the algorithmic TFLOP/s (linear 469.9 MFLOP per
    token + causal attention 2*d*L*len^2 per sequence)."""
    from mdlarc_scale_b200 import synthetic
    from mdlarc_scale_b200.engine import Engine, chunk_rows, plan_prefill
    from mdlarc_scale_b200.inference import pad_prompts
    dev = torch.device("cuda", 0)
    cfg, sd = model_state()
    cfg["max_seq_len"] = 16384
    engine = Engine(sd, cfg, dev)
    k = args.profile_prefill
    n = max(1, 64000 // (1863 * k + 932))
    tasks = synthetic.capped_tasks(3, n, k, k, 30, 30, None)
    prompts, positions = synthetic.prompts_for(tasks)
    ids, pos, mask = pad_prompts(prompts, positions, left=False)
    lens = mask.sum(axis=1)
    cap = 65536
    sess = engine.new_session(n, int(lens.max()) + 8, 8, cap, stop_on_end=False)
    plans = [plan_prefill(ids, pos, mask, r).to(dev) for r in chunk_rows(lens, cap)]
    ms = []
    for _ in range(args.warmup + args.steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for p in plans:
            sess.prefill(p, None)
        e1.record()
        e1.synchronize()
        ms.append(e0.elapsed_time(e1))
    sess.poll()
    t = float(np.mean(ms[args.warmup:])) / 1e3
    ntok = int(lens.sum())
    lin = ntok * 469.9e6
    att = float((2.0 * 1280 * 12 * lens.astype(np.float64) ** 2).sum())
    print(json.dumps({"profile": "prefill", "pairs": k, "sequences": n, "tokens": ntok, "max_len": int(lens.max()),
                      "ms": t * 1e3, "tokens_per_s": ntok / t, "linear_tflop": lin / 1e12, "attention_tflop": att / 1e12,
                      "tflops": (lin + att) / t / 1e12, "frac_of_bf16_burst_peak": (lin + att) / t / 1e12 / 1672.1}))


def profile_long_context(args):
    """One wave of the prefill-heavy large configuration end to end: `--profile-long` prompts of 5
    pairs of 30x30 grids + a 30x30 test input (10 247 tokens each), then `--max-new` greedy tokens with
    END suppressed.  Prints prefill and decode rates and the decode-attention bandwidth over the long
    cache (algorithmic bytes = cached positions x 61 440 B per sequence per step)."""
    from mdlarc_scale_b200 import synthetic
    from mdlarc_scale_b200.engine import Engine
    from mdlarc_scale_b200.inference import generate_tokens, pad_prompts
    dev = torch.device("cuda", 0)
    cfg, sd = model_state()
    cfg["max_seq_len"] = 16384
    engine = Engine(sd, cfg, dev)
    n = args.profile_long
    tasks = synthetic.capped_tasks(3, n, 5, 5, 30, 30, None)
    prompts, positions = synthetic.prompts_for(tasks)
    ids, pos, mask = pad_prompts(prompts, positions, left=False)
    lens = mask.sum(axis=1)
    generate_tokens(engine, ids[:2], pos[:2], mask[:2], None, 4, stop_on_end=False)   # warm-up

    def timed(max_new):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(dev)
        e0.record()
        tr = generate_tokens(engine, ids, pos, mask, None, max_new, stop_on_end=False)
        e1.record()
        e1.synchronize()
        del tr
        return e0.elapsed_time(e1) / 1e3

    t_prefill = timed(1)
    t_all = timed(MAX_NEW)
    t_decode = t_all - t_prefill
    steps = MAX_NEW - 1
    mean_len = float(lens.mean()) + steps / 2.0
    attn_bytes = n * mean_len * 61440.0 * steps
    print(json.dumps({"profile": "long context", "sequences": n, "prompt_tokens": int(lens.sum()),
                      "new_tokens": MAX_NEW, "prefill_s": t_prefill, "prefill_tokens_per_s": int(lens.sum()) / t_prefill,
                      "decode_s": t_decode, "ms_per_decode_step": t_decode / steps * 1e3,
                      "generated_tokens_per_s": n * MAX_NEW / t_all,
                      "kv_bytes_read_per_step": attn_bytes / steps,
                      "decode_step_gbs_counting_kv_only": attn_bytes / t_decode / 1e9}))


def profile_decode_small(args):
    """The decode step's kernels at the benchmark's batch (M = `--profile-decode-small` sequences, large
    model) on a deliberately small KV cache: 1 train pair of grids up to 3x3 (prompts of a few dozen
    tokens), 64 cache positions, 16 decode steps.  A few GB resident, so that multi-pass ncu captures
    of the length-independent kernels (residual GEMM, RMSNorm, head, decode_begin) stay short."""
    from mdlarc_scale_b200 import synthetic
    from mdlarc_scale_b200.engine import Engine
    from mdlarc_scale_b200.inference import generate_tokens, pad_prompts
    dev = torch.device("cuda", 0)
    cfg, sd = model_state()
    engine = Engine(sd, cfg, dev)
    n = args.profile_decode_small
    tasks = synthetic.capped_tasks(5, n, 1, 1, 1, 3, None)
    prompts, positions = synthetic.prompts_for(tasks)
    ids, pos, mask = pad_prompts(prompts, positions, left=False)
    ms = []
    for _ in range(args.warmup + args.steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        tr = generate_tokens(engine, ids, pos, mask, None, 16, stop_on_end=False)
        e1.record()
        e1.synchronize()
        ms.append(e0.elapsed_time(e1))
        del tr
    print(json.dumps({"profile": "decode step, small cache", "sequences": n, "max_prompt": int(mask.sum(axis=1).max()),
                      "decode_steps": 15, "ms_per_call": ms}))


def profile_fanout(args):
    """The fan-out kernels at the size of the voting configuration (400 synthetic tasks x 8 dihedral
    x 20 colour permutations = 64 000 variants), each as ONE launch through the C ABI with its
    index arrays already on the device: device-side prompt construction of all variants, and
    candidate canonicalisation of 64 000 rows of 931 tokens.  Prints the algorithmic bytes (arrays
    written / read once) and the achieved bandwidth, plus the host-side cost of `TaskTable`."""
    import ctypes as C
    from mdlarc_scale_b200 import _lib, fanout, synthetic
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    tasks = synthetic.capped_tasks(2, args.profile_fanout, 2, 4, 1, 30, 2048)
    t0 = time.perf_counter()
    table = fanout.TaskTable(tasks, dev, num_color_perms=20)
    vt = table.variants()
    t_table = time.perf_counter() - t0
    n = len(vt)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def up(a):
        return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)

    def timed(fn):
        best = None
        for _ in range(4):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(dev)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            best = e0.elapsed_time(e1) if best is None else min(best, e0.elapsed_time(e1))
        return best

    tok_off = np.concatenate([[0], np.cumsum(vt.length)]).astype(np.int64)
    total = int(tok_off[-1])
    d_tpl, d_dih, d_perm, d_off = up(vt.template), up(vt.dihedral), up(vt.perm), up(tok_off)
    out = torch.empty((8, total), dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    pb = _lib.PromptBuildArgs(
        n_variants=n, n_perms=20, d_cells=table.d_cells.data_ptr(), d_grid_off=table.d_grid_off.data_ptr(),
        d_grid_h=table.d_grid_h.data_ptr(), d_grid_w=table.d_grid_w.data_ptr(), d_tpl_off=table.d_tpl_off.data_ptr(),
        d_tpl_grid=table.d_tpl_grid.data_ptr(), d_perm_lut=table.d_perm_lut.data_ptr(),
        d_var_template=d_tpl.data_ptr(), d_var_dihedral=d_dih.data_ptr(), d_var_perm=d_perm.data_ptr(),
        d_var_tok_off=d_off.data_ptr(), d_var_seq=None, d_token_ids=out[0].data_ptr(), d_pos_xyz=out[1:4].data_ptr(),
        d_seq=out[4].data_ptr(), d_kv_slot=out[5].data_ptr(), d_kv_count=out[6].data_ptr(),
        d_kv_row=out[7].data_ptr(), d_status=status.data_ptr())
    build_ms = timed(lambda: _lib.check(lib.arcb_build_prompts(C.byref(pb), stream)))
    assert int(status.item()) == 0
    build_bytes = total * 32          # token id, 3 position words, seq, slot, count, scratch row
    del out
    # canonicalisation: well-formed generations (a transformed grid, END, then END padding)
    rng = np.random.default_rng(0)
    max_new = 931
    rows = np.full((n, max_new), 13, np.int32)
    for i in range(0, n, 160):
        g = rng.integers(0, 10, size=(int(rng.integers(1, 31)), int(rng.integers(1, 31))))
        t = np.concatenate([np.concatenate([r, [11]]) for r in g] + [[13]]).astype(np.int32)
        rows[i: i + 160, : len(t)] = t
    d_rows = torch.from_numpy(rows).to(dev)
    rec = torch.empty((n, fanout.RECORD_BYTES), dtype=torch.uint8, device=dev)
    d_test = up(table.tpl_test_grid[vt.template])
    ca = _lib.CandidateArgs(
        n_rows=n, max_new=max_new, d_tokens=d_rows.data_ptr(), d_row_dihedral=d_dih.data_ptr(),
        d_row_perm=d_perm.data_ptr(), d_perm_lut=table.d_perm_lut.data_ptr(), n_perms=20,
        d_row_test_grid=d_test.data_ptr(), d_cells=table.d_cells.data_ptr(), d_grid_off=table.d_grid_off.data_ptr(),
        d_grid_h=table.d_grid_h.data_ptr(), d_grid_w=table.d_grid_w.data_ptr(), d_records=rec.data_ptr())
    canon_ms = timed(lambda: _lib.check(lib.arcb_canonicalize_candidates(C.byref(ca), stream)))
    canon_bytes = n * (max_new * 4 + fanout.RECORD_BYTES)
    print(json.dumps({"profile": "fan-out kernels", "tasks": len(tasks), "variants": n, "prompt_tokens": total,
                      "table_upload_and_shapes_s": t_table,
                      "build_prompts": {"ms": build_ms, "bytes_written": build_bytes, "gbs": build_bytes / build_ms / 1e6},
                      "canonicalize": {"ms": canon_ms, "bytes_read_plus_written": canon_bytes,
                                       "gbs": canon_bytes / canon_ms / 1e6}}))


def torch_gpu_baseline_sample(dev, batch: int):
    """The reference's own generate_output (PyTorch eager: cuBLAS linears, SDPA attention, its Python
    decode loop) on THIS GPU in bf16, on one full step of the same workload (same generator, same
    sequences per step, same token budget, END suppressed).  A library-call baseline: what the
    hand-written kernels and the graph-captured step have to beat on equal hardware.  Returns None when
    the reference files are not present."""
    ref = _reference_model()
    if ref is None:
        return None
    model, generate_output = ref
    ids, pos, mask = make_batch(424242, batch)
    try:
        gpu_model = model.to(device=dev, dtype=torch.bfloat16)
        ids_t, pos_t, mask_t = (torch.from_numpy(a).to(dev) for a in (ids, pos, mask))
        with torch.no_grad():
            generate_output(gpu_model, ids_t[:8], pos_t[:8], None, mask_t[:8], max_new_tokens=4, stop_on_end=False)
            torch.cuda.synchronize(dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = generate_output(gpu_model, ids_t, pos_t, None, mask_t, max_new_tokens=MAX_NEW, stop_on_end=False)
            e1.record()
            e1.synchronize()
        dt = e0.elapsed_time(e1) / 1e3
        gen = out.shape[1] - ids.shape[1]
        res = {"value": batch * gen / dt, "unit": "tokens/s", "seconds": dt, "sequences": batch, "new_tokens": gen,
               "dtype": "bf16", "same_config": True,
               "what": "reference generate_output (src/inference.py), unmodified, PyTorch eager on this GPU, "
                       "inputs resident on the device, CUDA-event timed"}
        del out, ids_t, pos_t, mask_t
    except Exception as exc:  # e.g. out of memory for its zero-filled padded cache
        res = {"value": None, "error": f"{type(exc).__name__}: {str(exc)[:160]}"}
    finally:
        model.to(device="cpu", dtype=torch.float32)
        torch.cuda.empty_cache()
    return res


def prefill_heavy_sample(engine, dev, repeats: int = 3):
    """One prefill call of the prefill-heavy large configuration: 6 prompts of 5 pairs of 30x30 grids
    plus a 30x30 test input (10 247 tokens each, 61 482 packed tokens), timed with CUDA events.
    Algorithmic FLOPs: 469.9 MFLOP per token for the linear layers + 2 * d * L * len^2 per sequence for
    causal attention (only the causal half is counted)."""
    from mdlarc_scale_b200 import synthetic
    from mdlarc_scale_b200.engine import plan_prefill
    from mdlarc_scale_b200.inference import pad_prompts
    tasks = synthetic.capped_tasks(3, 6, 5, 5, 30, 30, None)
    prompts, positions = synthetic.prompts_for(tasks)
    ids, pos, mask = pad_prompts(prompts, positions, left=False)
    lens = mask.sum(axis=1)
    sess = engine.new_session(len(prompts), int(lens.max()) + 8, 8, 65536, stop_on_end=False)
    plan = plan_prefill(ids, pos, mask, np.arange(len(prompts))).to(dev)
    ms = []
    for i in range(1 + repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        sess.prefill(plan, None)
        e1.record()
        e1.synchronize()
        if i > 0:
            ms.append(e0.elapsed_time(e1))
    # the same call once more after a pause, i.e. at the clocks a call made on an idle GPU sees: the
    # repeats above follow the benchmark loop and run power-capped, which is what the sustained peak is
    # for; the burst peak (a GEMM timed alone) is the fair denominator for this one
    torch.cuda.synchronize(dev)
    time.sleep(3.0)
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    sess.prefill(plan, None)
    c1.record()
    c1.synchronize()
    cold_ms = c0.elapsed_time(c1)
    sess.poll()
    sess.close()
    t = float(np.mean(ms)) / 1e3
    ntok = int(lens.sum())
    flop = ntok * LINEAR_FLOP_PER_TOKEN + float((2.0 * engine.d_model * engine.n_layers * lens.astype(np.float64) ** 2).sum())
    burst, sustained, kind = measured_tensor_peaks()
    return {"workload": "cfg3-large-prefill: one call of 6 prompts x 10247 tokens (5 pairs of 30x30 + test input)",
            "tokens": ntok, "ms": t * 1e3, "ms_all": [round(x, 3) for x in ms], "tokens_per_s_per_gpu": ntok / t,
            "algorithmic_tflop": flop / 1e12, "tflops": flop / t / 1e12,
            "frac_of_bf16_burst_peak": flop / t / 1e12 / burst, "frac_of_bf16_sustained_peak": flop / t / 1e12 / sustained,
            "after_3s_idle": {"ms": cold_ms, "tflops": flop / cold_ms / 1e9,
                              "frac_of_bf16_burst_peak": flop / cold_ms / 1e9 / burst},
            "peak_kind": kind, "peaks_tflops": {"burst": burst, "sustained": sustained}}


def vote_pipeline_sample(rank, world, dev, dist, n_tasks: int = 8, perms: int = 20):
    """The voting configuration's multi-GPU pipeline on a bounded sample: medium model, n_tasks x 8
    dihedral x perms colour permutations variants dealt to the ranks by length-sorted round-robin,
    prompts built and candidates canonicalised on the device, ONE all-gather of the candidate
    records, AAIVR vote on every rank.  The vote digest must not depend on the number of ranks."""
    import hashlib
    from mdlarc_scale_b200 import fanout, sharding, synthetic
    from mdlarc_scale_b200.engine import Engine
    cfg, sd = synthetic.seeded_weights("medium", 0, 8.0)
    engine = Engine(sd, cfg, dev)
    tasks = synthetic.capped_tasks(2, n_tasks, 2, 4, 1, 30, 2048)
    table = fanout.TaskTable(tasks, dev, num_color_perms=perms)
    vt = table.variants()
    if dist is not None:
        # one untimed collective of the same shape first: the first all-gather of a new size pays NCCL's
        # channel set-up (tens of ms), which is not the cost of the pipeline's collective
        per = sharding.rows_per_rank(len(vt), world)
        warm = torch.zeros((world * per, fanout.RECORD_BYTES), dtype=torch.uint8, device=dev)
        for _ in range(2):
            dist.all_gather_into_tensor(warm, warm[rank * per: (rank + 1) * per])
        del warm
    torch.cuda.synchronize(dev)
    if dist is not None:
        dist.barrier()
    timing = {}
    t0 = time.perf_counter()
    records = sharding.generate_sharded_records(table, vt, MAX_NEW_FULL, rank, world, engine, timing=timing)
    torch.cuda.synchronize(dev)
    t_gen = time.perf_counter() - t0
    t1 = time.perf_counter()
    votes = fanout.vote_records(records, vt, top_k=2, seed=7)
    t_vote = time.perf_counter() - t1
    digest = hashlib.sha256(json.dumps(sorted((list(k), v) for k, v in votes.items())).encode()).hexdigest()
    gen = fanout.record_fields(records)[4].astype(np.int64)
    per_rank = [int((vt.length[idx].astype(np.int64) + gen[idx]).sum()) for idx in sharding.assign(vt.length, world)]
    ag_ms = float(timing.get("all_gather_ms", 0.0))
    if dist is not None:
        t = torch.tensor([t_gen, ag_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_gen, ag_ms = float(t[0].item()), float(t[1].item())
    engine.close()
    torch.cuda.empty_cache()
    return {"workload": f"cfg2-medium sample: {n_tasks} tasks x 8 dihedral x {perms} colour permutations = {len(vt)} variants, "
                        f"prompts <= 2048 tokens, greedy to END or {MAX_NEW_FULL} tokens",
            "n_gpus": world, "variants": int(len(vt)), "generate_and_gather_s": t_gen,
            "all_gather_ms": ag_ms, "all_gather_bytes": int(timing.get("gather_bytes", 0)),
            "wait_for_slowest_rank_ms": float(timing.get("wait_for_slowest_rank_ms", 0.0)),
            "vote_s": t_vote, "generated_tokens": int(gen.sum()), "generated_tokens_per_s": float(gen.sum()) / t_gen,
            "rank_tokens_max_over_mean": max(per_rank) / (sum(per_rank) / len(per_rank)),
            "tasks_with_votes": sum(1 for v in votes.values() if v), "votes_sha256": digest}



def run_ours(args, rank, world, local_rank):
    from mdlarc_scale_b200 import _lib
    from mdlarc_scale_b200.engine import Engine, chunk_rows, plan_prefill
    from mdlarc_scale_b200.inference import generate_output

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    cfg, sd = model_state()
    engine = Engine(sd, cfg, dev)
    lib = engine.lib
    B = args.batch
    n_total = args.warmup + args.steps
    batches = [make_batch(10_000 * rank + i, B) for i in range(n_total)]
    prefill_cap = 65536
    session = engine.new_session(B, KV_POSITIONS, MAX_NEW, prefill_cap, stop_on_end=False)
    session_pitch = session.t_max   # rows reserved per (sequence, head): the capacity rounded up to 16 mod 32

    def upload(batch):
        ids, pos, mask = batch
        lens = mask.sum(axis=1)
        return [plan_prefill(ids, pos, mask, rows).to(dev) for rows in chunk_rows(lens, prefill_cap)], lens

    def device_step(plans):
        for p in plans:
            session.prefill(p, None)
        session.decode(MAX_NEW - 1)

    def barrier():
        torch.cuda.synchronize(dev)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- device-timed value: inputs resident in HBM ----
    resident = [upload(b) for b in batches]
    for i in range(args.warmup):
        device_step(resident[i][0])
    session.poll()
    barrier()
    lib.arcb_launch_count(1)
    sampler = ClockSampler(local_rank)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with sampler:
        e0.record()
        for i in range(args.warmup, n_total):
            device_step(resident[i][0])
        e1.record()
        barrier()
    launches = int(lib.arcb_launch_count(0))
    session.poll()
    # live sample from inside the timed region: the layer-0 attention launch of the LAST decode step
    # (event nodes in the step graph); every row is then at prompt length + MAX_NEW - 1 cached positions
    try:
        live_ms = session.attention_probe_ms()
    except RuntimeError:
        live_ms = float("nan")
    live_bytes = float((resident[n_total - 1][1] + (MAX_NEW - 1)).sum()) * engine.n_heads * 64 * 2 * 2
    dt = e0.elapsed_time(e1) / 1e3
    prefill_tokens = int(sum(int(r[1].sum()) for r in resident[args.warmup:]))
    # prefill share, device-timed on the same inputs (one extra untimed-for-value pass)
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    for p in resident[-1][0]:
        session.prefill(p, None)
    p1.record()
    p1.synchronize()
    prefill_s = p0.elapsed_time(p1) / 1e3
    prefill_tok_s = int(resident[-1][1].sum()) / prefill_s
    session.decode(8)
    attn_gbs, attn_ms, attn_bytes = attention_roofline(engine, session, resident[-1][1])
    lens_last = resident[-1][1]
    del resident

    # ---- end to end through the public API: pinned host tensors in, host tokens out ----
    session.close()
    del session
    torch.cuda.empty_cache()
    if args.no_e2e:
        if rank == 0:
            print(json.dumps({"profiling_run": True, "value": world * args.steps * B * MAX_NEW / dt,
                              "attn_gbs": attn_gbs, "prefill_tok_s": prefill_tok_s, "gpu_launches": launches}))
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return
    host = []
    for ids, pos, mask in batches:
        host.append((torch.from_numpy(ids).pin_memory(), torch.from_numpy(pos).pin_memory(),
                     torch.from_numpy(mask).pin_memory()))
    h2d = d2h = 0
    for i in range(min(args.warmup, 1)):
        generate_output(engine, *host[i][:2], None, host[i][2], max_new_tokens=MAX_NEW, stop_on_end=False)
    barrier()
    t0 = time.perf_counter()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    for i in range(args.warmup, n_total):
        ids_t, pos_t, mask_t = host[i]
        out = generate_output(engine, ids_t, pos_t, None, mask_t, max_new_tokens=MAX_NEW, stop_on_end=False)
        assert out.device.type == "cpu" and out.shape[1] == ids_t.shape[1] + MAX_NEW
        n_valid = int(mask_t.sum())
        h2d += n_valid * 4 * 7 + B * 4 * 6  # packed ids, xyz, seq, slot, count (+ per-sequence arrays)
        d2h += B * MAX_NEW * 4
    g1.record()
    barrier()
    e2e_dt = max(time.perf_counter() - t0, g0.elapsed_time(g1) / 1e3)

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    dt = max_over_ranks(dt)
    e2e_dt = max_over_ranks(e2e_dt)
    # outside every timed region: the prefill-heavy configuration's prefill call (rank 0) and the voting
    # configuration's sharded pipeline (all ranks)
    del host
    torch.cuda.empty_cache()
    extras = {}
    if not args.no_extras:
        if rank == 0:
            extras["prefill_heavy"] = prefill_heavy_sample(engine, dev)
        engine.close()
        torch.cuda.empty_cache()
        extras["vote_pipeline"] = vote_pipeline_sample(rank, world, dev, dist)
        if rank == 0 and world == 1 and not args.no_torch_gpu:
            tg = torch_gpu_baseline_sample(dev, B)
            if tg is not None:
                extras["torch_gpu_baseline"] = tg
    gen_tokens = world * args.steps * B * MAX_NEW
    clocks = sampler.summary()
    if rank == 0:
        peak, peak_kind = measured_peaks()
        line = {
            "metric": "generated tokens/s", "value": gen_tokens / dt, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000 * dt / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "cfg4-large-decode", "model": MODEL_SIZE, "sequences_per_gpu_per_step": B,
                       "new_tokens": MAX_NEW, "kv_positions": KV_POSITIONS, "kv_row_pitch": session_pitch, "stop_on_end": False,
                       "activations": "f16 operands, bf16 weights + KV cache, f32 accumulate/residual",
                       "l2": "inputs larger than L2 (KV cache %.1f GB per GPU)" % (B * session_pitch * engine.kv_bytes_per_position() / 1e9),
                       "parallelism": f"dp{world} (independent sequence shards)"},
            "e2e": {"value": gen_tokens / e2e_dt, "unit": "tokens/s", "h2d_bytes_per_step": h2d // args.steps,
                    "d2h_bytes_per_step": d2h // args.steps},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": attn_gbs, "peak": peak, "unit": "GB/s",
                         "frac": attn_gbs / peak, "traffic": attn_bytes * ATTN_TRAFFIC_PER_ALGORITHMIC_BYTE, "peak_kind": peak_kind,
                         "kernel": "attn_stream_coop_kernel (decode attention)", "ms_per_launch": attn_ms,
                         "algorithmic_bytes_per_launch": attn_bytes,
                         "in_graph_sample": {"what": "layer-0 attention launch of the last timed decode step, "
                                                     "CUDA event nodes inside the step graph",
                                             "ms": live_ms, "algorithmic_bytes": live_bytes,
                                             "gbs": live_bytes / live_ms / 1e6}},
            "prefill": {"tokens_per_s_per_gpu": prefill_tok_s, "tokens_per_step": prefill_tokens // args.steps},
        }
        line.update(extras)
        if not args.no_cpu and world == 1:
            torch.set_num_threads(os.cpu_count() or 1)
            v, cdt, kind, mean_cache = cpu_generate_sample(args.cpu_seqs, args.cpu_steps, 777)
            line["cpu_baseline"] = {
                "value": v, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": kind,
                "sample": _cpu_sample_text(args.cpu_seqs, args.cpu_steps, kind, mean_cache, cdt)}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    global MAX_NEW
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1024, help="sequences per GPU per step")
    ap.add_argument("--cpu-seqs", type=int, default=32)
    ap.add_argument("--cpu-steps", type=int, default=112)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiling runs)")
    ap.add_argument("--no-torch-gpu", action="store_true",
                    help="skip the reference's own PyTorch path timed on this GPU (N = 1 only)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the prefill-heavy prefill call and the sharded vote pipeline sample")
    ap.add_argument("--profile-attn", type=int, default=0, metavar="T",
                    help="only run 4 standalone decode-attention launches over T cached positions (ncu target)")
    ap.add_argument("--profile-attn-spread", type=int, default=0, metavar="S",
                    help="with --profile-attn: lengths uniform in T - S .. T + S instead of T everywhere")
    ap.add_argument("--profile-attn-pitch", type=int, default=0, metavar="ROWS",
                    help="with --profile-attn: cache capacity (rows per sequence and head) when larger than T + S")
    ap.add_argument("--profile-prefill", type=int, default=0, metavar="PAIRS",
                    help="only time the prefill of ~64k tokens of prompts with PAIRS 30x30 train pairs")
    ap.add_argument("--profile-fanout", type=int, default=0, metavar="TASKS",
                    help="only time the fan-out kernels for TASKS synthetic tasks x 8 x 20 variants")
    ap.add_argument("--profile-long", type=int, default=0, metavar="SEQS",
                    help="only run one wave of SEQS 10 247-token prompts + --max-new tokens (long-context decode)")
    ap.add_argument("--profile-decode-small", type=int, default=0, metavar="SEQS",
                    help="only run prefill + 15 decode steps of SEQS tiny prompts on a 64-position cache (ncu target)")
    ap.add_argument("--max-new", type=int, default=MAX_NEW,
                    help="tokens generated per sequence (the workload uses 931; smaller only for profiling)")
    args = ap.parse_args()
    MAX_NEW = args.max_new
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        # started without a launcher: re-run under torchrun, one rank per GPU, rendezvous on 127.0.0.1
        port = 29500 + os.getpid() % 1000
        os.execvp(sys.executable, [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                                   f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1",
                                   "--master-port", str(port), os.path.abspath(__file__), *sys.argv[1:]])
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200 GPU (the product path has no CPU fallback)")
    if args.profile_attn > 0:
        profile_attention(args)
        return
    if args.profile_prefill > 0:
        profile_prefill(args)
        return
    if args.profile_long > 0:
        profile_long_context(args)
        return
    if args.profile_fanout > 0:
        profile_fanout(args)
        return
    if args.profile_decode_small > 0:
        profile_decode_small(args)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
