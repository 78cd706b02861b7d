"""The allocation-free decode-attention entry point against the regular one.

Callers that may not allocate on the hot path (fixed memory pools, plugins inside another
framework's allocator) use arcb_op_decode_attention_static, whose split-K scratch is an array
built into the library.  It must give what arcb_op_decode_attention gives with a caller-provided
scratch, also on a second call that finds the first call's leftovers in the shared array.
This file sorts last so that a run stopping at the first failure has already run everything else.
"""
import pytest
import torch

from gpu_util import have_b200, stream, to_act
from mdlarc_scale_b200 import _lib

pytestmark = pytest.mark.gpu


def _case(seed, B, H, T, lens, fmt):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = to_act(torch.randn(B, H, 64, device="cuda", generator=g), fmt)
    k = torch.randn(B, H, T, 64, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(B, H, T, 64, device="cuda", generator=g).to(torch.bfloat16)
    return q, k, v, torch.tensor(lens, dtype=torch.int32, device="cuda")


def test_static_scratch_entry_matches_regular_entry_twice():
    if not have_b200():
        pytest.fail("this test needs a B200 (compute capability 10.x)")
    lib = _lib.load()
    fmt = _lib.ACT_F16
    # two different calls in a row: the second is smaller, so stale records of the first remain
    # in the shared array next to the ones it overwrites
    for seed, (B, H, T, splits, lens) in enumerate([(6, 4, 400, 8, [400, 1, 33, 257, 128, 64]),
                                                    (3, 4, 200, 3, [7, 200, 90])]):
        q, k, v, lens_t = _case(seed, B, H, T, lens, fmt)
        want = torch.full((B, H, 64), float("nan"), device="cuda", dtype=q.dtype)
        got = torch.full((B, H, 64), float("nan"), device="cuda", dtype=q.dtype)
        scratch = torch.empty(lib.arcb_attn_scratch_bytes(B, H, splits), dtype=torch.uint8, device="cuda")
        _lib.check(lib.arcb_op_decode_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), want.data_ptr(), None,
                                                lens_t.data_ptr(), None, B, H, T, splits, scratch.data_ptr(), fmt,
                                                stream()))
        _lib.check(lib.arcb_op_decode_attention_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), got.data_ptr(),
                                                       None, lens_t.data_ptr(), None, B, H, T, splits, fmt,
                                                       stream()))
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        # same tolerance as the decode-attention kernel test (half outputs)
        assert torch.allclose(got.float(), want.float(), rtol=2 ** -10, atol=2e-3)
        # and directly against an fp32 softmax attention over each item's visible prefix
        for b, n in enumerate(lens):
            att = torch.softmax(torch.einsum("hd,htd->ht", q[b].float(), k[b, :, :n].float()) / 8.0, dim=-1)
            ref = torch.einsum("ht,htd->hd", att, v[b, :, :n].float())
            assert torch.allclose(got[b].float(), ref, rtol=2 ** -9, atol=3e-3), b


def test_static_scratch_entry_rejects_oversize():
    if not have_b200():
        pytest.fail("this test needs a B200 (compute capability 10.x)")
    lib = _lib.load()
    q, k, v, lens_t = _case(0, 2, 2, 16, [16, 16], _lib.ACT_F16)
    out = torch.empty_like(q)
    too_many_items = _lib.STATIC_ATTN_MAX_RECORDS // (2 * 4) + 1
    rc = lib.arcb_op_decode_attention_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), None,
                                             lens_t.data_ptr(), None, too_many_items, 2, 16, 4, _lib.ACT_F16,
                                             stream())
    assert rc == _lib.E_ARG
    assert b"ARCB_STATIC_ATTN_MAX_RECORDS" in lib.arcb_last_error()
