"""Each CUDA kernel, called through the C ABI, against a plain fp32 torch reference of the same op."""
import math

import pytest
import torch

from gpu_util import have_b200, stream, to_act
from mdlarc_scale_b200 import _lib

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    if not have_b200():
        pytest.fail("these tests need a B200 (compute capability 10.x)")
    return _lib.load()


@pytest.mark.parametrize("fmt", [_lib.ACT_F16, _lib.ACT_BF16])
@pytest.mark.parametrize("rows,d", [(1, 256), (7, 768), (130, 1280)])
def test_rmsnorm(lib, fmt, rows, d):
    g = torch.Generator(device="cuda").manual_seed(rows * d)
    x = torch.randn(rows, d, device="cuda", generator=g) * 3
    w = torch.randn(d, device="cuda", generator=g)
    out = torch.empty(rows, d, device="cuda", dtype=torch.float16 if fmt == _lib.ACT_F16 else torch.bfloat16)
    _lib.check(lib.arcb_op_rmsnorm(x.data_ptr(), w.data_ptr(), out.data_ptr(), rows, d, 1e-5, fmt, stream()))
    ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w
    eps = 2 ** -10 if fmt == _lib.ACT_F16 else 2 ** -7
    assert torch.allclose(out.float(), ref, rtol=eps, atol=1e-4)


@pytest.mark.parametrize("path", [_lib.GEMM_SIMT, _lib.GEMM_TC, _lib.GEMM_TC_1CTA, _lib.GEMM_TC_2CTA],
                         ids=["simt", "tc", "tc1cta", "tc2cta"])
@pytest.mark.parametrize("fmt", [_lib.ACT_BF16, _lib.ACT_F16], ids=["bf16", "f16"])
@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 768, 256), (33, 256, 704), (128, 384, 128),
                                   (300, 1408, 256), (1000, 1280, 3392),
                                   (2048, 3840, 256), (4000, 6784, 128), (20000, 1280, 192)])
def test_gemm(lib, path, fmt, M, N, K):
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = to_act(torch.randn(M, K, device="cuda", generator=g), fmt)
    w = to_act((torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16).float(), fmt)
    y = torch.full((M, N), float("nan"), device="cuda")
    _lib.check(lib.arcb_op_gemm(a.data_ptr(), w.data_ptr(), y.data_ptr(), M, N, K, fmt, path, stream()))
    torch.cuda.synchronize()
    ref = a.double() @ w.double().t()
    err = (y.double() - ref).abs().max().item()
    assert err < 2e-4 * math.sqrt(K / 64), f"max abs err {err}"


@pytest.mark.parametrize("path", [_lib.GEMM_SIMT, _lib.GEMM_TC_1CTA, _lib.GEMM_TC_2CTA], ids=["simt", "tc1cta", "tc2cta"])
@pytest.mark.parametrize("with_bias", [False, True])
@pytest.mark.parametrize("M,N,K", [(33, 256, 128), (129, 384, 704), (300, 1280, 256), (1000, 1280, 3392),
                                   (1024, 768, 768), (20001, 1280, 192)])
def test_gemm_residual(lib, path, with_bias, M, N, K):
    """x += A W^T (+ bias): the residual epilogue (bulk tensor reduce on the tensor-core kernels),
    row counts that leave a partial last tile, bitwise identical when repeated."""
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = to_act(torch.randn(M, K, device="cuda", generator=g), _lib.ACT_F16)
    w = to_act((torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16).float(), _lib.ACT_F16)
    bias = torch.randn(N, device="cuda", generator=g) if with_bias else None
    x0 = torch.randn(M + 3, N, device="cuda", generator=g)     # three guard rows after the last one
    outs = []
    for _ in range(2):
        x = x0.clone()
        _lib.check(lib.arcb_op_gemm_residual(a.data_ptr(), w.data_ptr(), bias.data_ptr() if with_bias else None,
                                             x.data_ptr(), M, N, K, _lib.ACT_F16, path, stream()))
        torch.cuda.synchronize()
        outs.append(x)
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(outs[0][M:], x0[M:])                    # rows beyond M are untouched
    ref = x0[:M].double() + a.double() @ w.double().t() + (bias.double() if with_bias else 0.0)
    err = (outs[0][:M].double() - ref).abs().max().item()
    assert err < 2e-4 * math.sqrt(K / 64) + 1e-5, f"max abs err {err}"


@pytest.mark.parametrize("with_bias", [False, True])
@pytest.mark.parametrize("M,N,K", [(1024, 1280, 1280), (1024, 1280, 3392), (1000, 1280, 3392), (600, 1024, 1024),
                                   (1024, 1024, 2752), (333, 1280, 1280)])
def test_gemm_residual_split_k(lib, with_bias, M, N, K):
    """The decode step's few-row residual GEMMs through the split-K kernel (pairs of CTAs, half of K
    each, fixed-order combine through a scratch, one reduce-add per element): against fp64, rows beyond
    M untouched, bitwise identical when repeated (also with a scratch full of garbage)."""
    nbytes = lib.arcb_gemm_splitk_scratch_bytes(M, N, K)
    assert nbytes == ((M + 127) // 128) * 128 * N * 4, "these shapes are the ones the kernel is meant for"
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = to_act(torch.randn(M, K, device="cuda", generator=g), _lib.ACT_F16)
    w = to_act((torch.randn(N, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16).float(), _lib.ACT_F16)
    bias = torch.randn(N, device="cuda", generator=g) if with_bias else None
    x0 = torch.randn(M + 3, N, device="cuda", generator=g)
    outs = []
    for fill in (0.0, float("nan")):
        scratch = torch.full((nbytes // 4,), fill, device="cuda")
        x = x0.clone()
        _lib.check(lib.arcb_op_gemm_residual_splitk(a.data_ptr(), w.data_ptr(), bias.data_ptr() if with_bias else None,
                                                    x.data_ptr(), M, N, K, _lib.ACT_F16, scratch.data_ptr(), stream()))
        torch.cuda.synchronize()
        outs.append(x)
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(outs[0][M:], x0[M:])
    ref = x0[:M].double() + a.double() @ w.double().t() + (bias.double() if with_bias else 0.0)
    err = (outs[0][:M].double() - ref).abs().max().item()
    assert err < 2e-4 * math.sqrt(K / 64) + 1e-5, f"max abs err {err}"
    # shapes that already fill the machine, or whose K is short, are refused
    assert lib.arcb_gemm_splitk_scratch_bytes(20000, 1280, 1280) == 0
    assert lib.arcb_gemm_splitk_scratch_bytes(1024, 1280, 256) == 0


@pytest.mark.parametrize("splits", [1, 4, 7])
@pytest.mark.parametrize("fmt", [_lib.ACT_F16, _lib.ACT_BF16])
def test_decode_attention(lib, splits, fmt):
    B, H, T = 5, 4, 300
    g = torch.Generator(device="cuda").manual_seed(splits)
    q = to_act(torch.randn(B, H, 64, device="cuda", generator=g), fmt)
    k = torch.randn(B, H, T, 64, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(B, H, T, 64, device="cuda", generator=g).to(torch.bfloat16)
    lens = torch.tensor([1, 17, 300, 64, 0], dtype=torch.int32, device="cuda")
    seqs = torch.tensor([4, 3, 2, 1, 0], dtype=torch.int32, device="cuda")
    out = torch.full((B, H, 64), float("nan"), device="cuda", dtype=q.dtype)
    scratch = torch.empty(max(1, lib.arcb_attn_scratch_bytes(B, H, splits)), dtype=torch.uint8, device="cuda")
    _lib.check(lib.arcb_op_decode_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                            seqs.data_ptr(), lens.data_ptr(), None, B, H, T, splits,
                                            scratch.data_ptr(), fmt, stream()))
    torch.cuda.synchronize()
    for i in range(B):
        n, s = int(lens[i]), int(seqs[i])
        if n == 0:
            assert torch.all(out[i] == 0)  # no visible key: zeros, like the reference's CPU attention
            continue
        sc = torch.einsum("hd,htd->ht", q[i].float(), k[s, :, :n].float()) / 8.0
        ref = torch.einsum("ht,htd->hd", torch.softmax(sc, -1), v[s, :, :n].float())
        eps = 2 ** -10 if fmt == _lib.ACT_F16 else 2 ** -7
        assert torch.allclose(out[i].float(), ref, rtol=eps, atol=2e-3), (i, (out[i].float() - ref).abs().max())


@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("fmt", [_lib.ACT_F16, _lib.ACT_BF16])
def test_decode_attention_many_items(lib, splits, fmt):
    """Launches with at least 296 (item, head, split) work items run the cooperative kernel (eight
    warps per work item, merged through shared memory): ragged lengths around the 32-row and 256-row
    slice boundaries, empty and skipped items, permuted cache rows."""
    B, H, T = 24, 20, 700
    g = torch.Generator(device="cuda").manual_seed(10 + splits)
    q = to_act(torch.randn(B, H, 64, device="cuda", generator=g), fmt)
    k = torch.randn(B, H, T, 64, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(B, H, T, 64, device="cuda", generator=g).to(torch.bfloat16)
    lens_l = [1, 31, 32, 33, 255, 256, 257, 700, 0, 511, 513, 64, 96, 300, 699, 2, 16, 48, 128, 384, 640, 5, 650, 289]
    lens = torch.tensor(lens_l, dtype=torch.int32, device="cuda")
    seqs = torch.randperm(B, device="cuda", generator=g).to(torch.int32)
    skip = torch.zeros(B, dtype=torch.uint8, device="cuda")
    skip[7] = 1
    out = torch.full((B, H, 64), float("nan"), device="cuda", dtype=q.dtype)
    scratch = torch.empty(max(1, lib.arcb_attn_scratch_bytes(B, H, splits)), dtype=torch.uint8, device="cuda")
    _lib.check(lib.arcb_op_decode_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                            seqs.data_ptr(), lens.data_ptr(), skip.data_ptr(), B, H, T, splits,
                                            scratch.data_ptr(), fmt, stream()))
    torch.cuda.synchronize()
    eps = 2 ** -10 if fmt == _lib.ACT_F16 else 2 ** -7
    for i in range(B):
        n, s = lens_l[i], int(seqs[i])
        if n == 0 or i == 7:
            assert torch.all(out[i] == 0)
            continue
        sc = torch.einsum("hd,htd->ht", q[i].float(), k[s, :, :n].float()) / 8.0
        ref = torch.einsum("ht,htd->hd", torch.softmax(sc, -1), v[s, :, :n].float())
        assert torch.allclose(out[i].float(), ref, rtol=eps, atol=2e-3), (i, n, (out[i].float() - ref).abs().max())


def test_head_logits_argmax(lib):
    rows, d = 37, 1280
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(64, d, device="cuda", generator=g)
    idx = torch.randperm(64, device="cuda", generator=g)[:rows].to(torch.int32)
    lnf = torch.randn(d, device="cuda", generator=g)
    head = torch.randn(14, d, device="cuda", generator=g) * 0.05
    logits = torch.empty(rows, 14, device="cuda")
    am = torch.empty(rows, dtype=torch.int32, device="cuda")
    _lib.check(lib.arcb_op_head(x.data_ptr(), idx.data_ptr(), lnf.data_ptr(), head.data_ptr(), logits.data_ptr(),
                                am.data_ptr(), rows, d, 1e-5, stream()))
    xs = x[idx.long()]
    ref = (xs * torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + 1e-5) * lnf) @ head.t()
    assert torch.allclose(logits, ref, atol=1e-4, rtol=1e-4)
    assert torch.equal(am.long(), logits.argmax(-1))
