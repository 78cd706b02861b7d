"""Seeded synthetic ARC-style tasks with the shapes and value distributions of the benchmark
configurations (stand-ins for the public task files, which are not available offline).

Grid height and width are uniform in [lo, hi]; a cell is 0 with probability 0.6, otherwise
uniform in 1..9.  A task has k train pairs and one test input.
"""
from __future__ import annotations

import numpy as np

from .data import DIHEDRAL_TRANSFORMS, compute_positions_3d, encode_example


def random_grid(rng: np.random.Generator, lo: int, hi: int) -> list[list[int]]:
    h = int(rng.integers(lo, hi + 1))
    w = int(rng.integers(lo, hi + 1))
    zero = rng.random((h, w)) < 0.6
    colours = rng.integers(1, 10, size=(h, w))
    return np.where(zero, 0, colours).astype(np.int64).tolist()


def random_task(rng: np.random.Generator, k_lo: int, k_hi: int, lo: int, hi: int) -> dict:
    k = int(rng.integers(k_lo, k_hi + 1))
    train = [{"input": random_grid(rng, lo, hi), "output": random_grid(rng, lo, hi)} for _ in range(k)]
    return {"train": train, "test": [{"input": random_grid(rng, lo, hi)}]}


def task_prompt(task: dict, test_idx: int = 0, dihedral_idx: int = 0) -> list[int]:
    """START in NEWLINE... IO_SEP out ... END per train pair, then the test input and IO_SEP."""
    f = DIHEDRAL_TRANSFORMS[dihedral_idx]
    toks: list[int] = []
    for p in task["train"]:
        toks += encode_example(f(p["input"]), f(p["output"]))
    toks += encode_example(f(task["test"][test_idx]["input"]), None)
    return toks


def capped_tasks(seed: int, n_tasks: int, k_lo: int, k_hi: int, lo: int, hi: int, cap: int | None) -> list[dict]:
    """n_tasks tasks; any whose identity-orientation prompt exceeds ``cap`` tokens is resampled."""
    rng = np.random.default_rng(seed)
    out = []
    while len(out) < n_tasks:
        t = random_task(rng, k_lo, k_hi, lo, hi)
        if cap is None or len(task_prompt(t)) <= cap:
            out.append(t)
    return out


def prompts_for(tasks: list[dict], dihedrals=(0,)) -> tuple[list[list[int]], list[np.ndarray]]:
    prompts, positions = [], []
    for t in tasks:
        for d in dihedrals:
            toks = task_prompt(t, 0, d)
            prompts.append(toks)
            positions.append(compute_positions_3d(toks))
    return prompts, positions


# The five benchmark configurations: model size and prompt generator.
CONFIGS = {
    0: dict(name="cfg0-tiny-8tasks", size="tiny", n_tasks=8, k=(2, 4), hw=(1, 30), cap=2048, dihedrals=(0,)),
    1: dict(name="cfg1-small-16x8", size="small", n_tasks=16, k=(2, 4), hw=(1, 30), cap=2048,
            dihedrals=tuple(range(8))),
    2: dict(name="cfg2-medium-400x8x20", size="medium", n_tasks=400, k=(2, 4), hw=(1, 30), cap=2048,
            dihedrals=tuple(range(8)), color_perms=20),
    3: dict(name="cfg3-large-prefill", size="large", n_tasks=256, k=(5, 5), hw=(30, 30), cap=None, dihedrals=(0,)),
    4: dict(name="cfg4-large-decode", size="large", n_tasks=2048, k=(2, 2), hw=(3, 10), cap=None, dihedrals=(0,)),
}


def config_prompts(cfg_idx: int, n_tasks: int | None = None, seed: int | None = None):
    c = CONFIGS[cfg_idx]
    tasks = capped_tasks(cfg_idx if seed is None else seed, n_tasks or c["n_tasks"], c["k"][0], c["k"][1],
                         c["hw"][0], c["hw"][1], c["cap"])
    return tasks, prompts_for(tasks, c["dihedrals"])


def seeded_weights(size: str, seed: int = 0, embed_gain: float = 1.0):
    """Seeded random-init weights with the reference's distributions (src/transformer.py:547-560),
    rounded to bf16; ``embed_gain`` > 1 makes generations varied enough to reach END."""
    import math

    import torch
    dims = {"tiny": (256, 4, 4, 704), "small": (768, 12, 4, 2048), "medium": (1024, 16, 8, 2752),
            "large": (1280, 20, 12, 3392)}[size]
    d, h, L, dff = dims
    g = torch.Generator().manual_seed(seed)

    def xavier(o, i):
        return (torch.rand(o, i, generator=g) * 2 - 1) * math.sqrt(6.0 / (i + o))

    sd = {"token_embed.weight": torch.randn(14, d, generator=g) * 0.02 * embed_gain,
          "example_embed.weight": torch.randn(1280, d, generator=g) * 0.02}
    for l in range(L):
        p = f"blocks.{l}."
        sd[p + "ln1.weight"] = torch.ones(d)
        sd[p + "attn.qkv_proj.weight"] = xavier(3 * d, d)
        sd[p + "attn.out_proj.weight"] = xavier(d, d)
        sd[p + "ln2.weight"] = torch.ones(d)
        sd[p + "ffn.fc_gate.weight"] = xavier(dff, d)
        sd[p + "ffn.fc_gate.bias"] = torch.zeros(dff)
        sd[p + "ffn.fc_up.weight"] = xavier(dff, d)
        sd[p + "ffn.fc_up.bias"] = torch.zeros(dff)
        sd[p + "ffn.fc_down.weight"] = xavier(d, dff)
        sd[p + "ffn.fc_down.bias"] = torch.zeros(d)
    sd["ln_f.weight"] = torch.ones(d)
    sd["lm_head.weight"] = xavier(14, d)
    cfg = dict(d_model=d, n_heads=h, n_layers=L, d_ff=dff, vocab_size=14, max_seq_len=4096, num_examples=1280,
               max_x=32, max_y=32, max_z=8, rope_base=10000.0, norm_eps=1e-5, use_example_embedding=True)
    return cfg, {k: v.to(torch.bfloat16).float() for k, v in sd.items()}
