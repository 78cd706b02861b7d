"""Helpers shared by the GPU tests (the tests call the product through its C ABI)."""
import ctypes as C

import numpy as np
import torch

from mdlarc_scale_b200 import _lib


def have_b200() -> bool:
    if not torch.cuda.is_available():
        return False
    return torch.cuda.get_device_capability(0)[0] == 10


def to_act(x: torch.Tensor, fmt: int) -> torch.Tensor:
    return x.to(torch.float16 if fmt == _lib.ACT_F16 else torch.bfloat16)


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def first_end_trim(row, end=13):
    row = list(row)
    return row[: row.index(end) + 1] if end in row else row


def tokens_agree(got, want, ref_logits_per_step, tol):
    """Greedy tokens must be identical except at positions where the reference's own top-2
    logit margin is below ``tol`` (after such a position the sequences may diverge)."""
    for i, (g, w) in enumerate(zip(got, want)):
        if g == w:
            continue
        top2 = np.sort(np.asarray(ref_logits_per_step[i]))[-2:]
        return (top2[1] - top2[0]) < tol, i
    return True, -1
