"""GPU tests against the reference's OWN CUDA kernels (compiled for sm_100a from the
reference checkout into oracle/_ref/ by `make -C oracle ref`).  Skipped when that library
has not been built."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from layerstormgemmkernels_b200 import quantize as Q
from layerstormgemmkernels_b200.capi import GGUF_TYPES

pytestmark = pytest.mark.gpu
T = GGUF_TYPES
REF_TYPES = ["Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "Q8_0", "MXFP4"]  # no Q4_0 in the reference


@pytest.fixture(scope="module")
def ref():
    lib = oracle.ref_lib()
    if lib is None:
        pytest.skip("oracle/_ref/libref_gguf.so not built")
    return lib


@pytest.fixture(scope="module")
def ops():
    from layerstormgemmkernels_b200 import ops as _ops
    return _ops


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("M,K", [(1, 4096), (5, 512), (8, 14336), (33, 2048), (611, 4096)])   # the last: one lane per block, ragged last CTA
def test_q8_1_bit_exact_vs_reference_kernel(ref, ops, M, K):
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(K + M))
    x[0, :32] = 0
    x[-1, 5] = 1e4
    xb = x.to(torch.bfloat16).cuda()
    want = torch.zeros((M, K // 32, 36), dtype=torch.uint8, device="cuda")
    assert ref.ref_quantize_q8_1(_p(xb), _p(want), M, K, _stream()) == 0
    got = ops.quantize_q8_1(xb)
    torch.cuda.synchronize()
    assert torch.equal(got, want)


@pytest.mark.parametrize("name", REF_TYPES)
@pytest.mark.parametrize("M", [1, 3, 8, 12])
def test_mmvq_vs_reference_kernel(ref, ops, name, M):
    t = T[name]
    N, K = 320, 1024
    A = (torch.randn(M, K, generator=torch.Generator().manual_seed(M)) * 0.4).to(torch.bfloat16).cuda()
    W = torch.from_numpy(Q.random_gguf_weight(name, N, K, seed=42)).cuda()
    want = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    ws = torch.zeros((M * (K // 32) * 36,), dtype=torch.uint8, device="cuda")
    assert ref.ref_gguf_mmvq(M, N, K, _p(A), _p(W), _p(want), t, _p(ws), _stream()) == 0
    got32 = ops.gguf_mmvq(A, W, t, N, K, out_dtype=torch.float32)
    got16 = ops.gguf_mmvq(A, W, t, N, K)
    torch.cuda.synchronize()
    w = want.float()
    scale = w.abs().max().item()
    # north-star bound: max |y - ref| / max |ref| <= 1e-3 on the un-rounded result; the
    # reference output itself carries a bf16 rounding of up to half an ulp = 2^-8 relative.
    assert (got32 - w).abs().max().item() <= (1e-3 + 2.0 ** -8) * scale
    # bf16 vs bf16: at most one bf16 ulp apart anywhere
    assert (got16.float() - w).abs().max().item() <= 2.0 ** -7 * scale
    # and identical on (nearly) every element
    assert (got16 == want).float().mean().item() > 0.97


@pytest.mark.parametrize("name", REF_TYPES)
def test_dequant_gemm_vs_reference_kernel(ref, ops, name):
    t = T[name]
    for M in (4, 40):
        N, K = 96, 512
        A = (torch.randn(M, K, generator=torch.Generator().manual_seed(3)) * 0.4).to(torch.bfloat16).cuda()
        W = torch.from_numpy(Q.random_gguf_weight(name, N, K, seed=7)).cuda()
        want = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
        assert ref.ref_gguf_dequant_gemm(M, N, K, _p(A), _p(W), _p(want), t, _stream()) == 0
        got = ops.gguf_dequant_gemm(A, W, t, N, K)
        torch.cuda.synchronize()
        scale = want.float().abs().max().item()
        assert (got.float() - want.float()).abs().max().item() <= 2.0 ** -7 * scale
        assert (got == want).float().mean().item() > 0.97


# ---------------------------------------------------------------------------
# Single-problem NVFP4 operators (csrc/smxx/quant/bf16_to_nvfp4.cu, reformat_scales.cu,
# nvfp4_dequant_bf16.cu of the reference): bytes must be equal.
# ---------------------------------------------------------------------------
def _need(ref, name):
    if not hasattr(ref, name):
        pytest.skip(f"oracle/_ref/libref_gguf.so was built without {name}: rebuild it (make -C oracle ref)")
    return getattr(ref, name)


@pytest.mark.parametrize("M,K", [(1, 64), (7, 256), (130, 1024), (257, 4096)])
def test_bf16_to_nvfp4_bytes_equal_reference_kernel(ref, ops, M, K):
    fn = _need(ref, "ref_bf16_to_nvfp4")
    g = torch.Generator().manual_seed(M * 7 + K)
    x = (torch.randn(M, K, generator=g) * torch.exp(torch.randn(M, 1, generator=g))).to(torch.bfloat16).cuda()
    x[0, :16] = 0                                   # an all-zero group
    packed, scales = ops.bf16_to_nvfp4(x)
    want_p = torch.zeros_like(packed)
    want_s = torch.zeros_like(scales)
    assert fn(_p(x), _p(want_p), _p(want_s), M, 128, K, _stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(packed, want_p)
    assert torch.equal(scales, want_s)


@pytest.mark.parametrize("N,K", [(1, 64), (96, 256), (128, 1024), (300, 2048)])
def test_reformat_scales_bytes_equal_reference_kernel(ref, ops, N, K):
    fn = _need(ref, "ref_reformat_scales")
    g = torch.Generator().manual_seed(N + K)
    src = (torch.rand(N, K // 16, generator=g) * 500.0 - 5.0).cuda()      # below 0 and above 480 included
    src[0, 0] = 2.0 ** -10                                                  # rounds to zero or the smallest code
    got = ops.nvfp4_gemm_preprocess(src, N, K)
    want = torch.zeros_like(got)
    assert fn(ctypes.c_void_p(src.data_ptr()), _p(want), N, K // 16, 1, N, K, 0, _stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(got, want)


@pytest.mark.parametrize("N,K", [(1, 64), (33, 512), (256, 4096)])
def test_nvfp4_dequant_bf16_equal_reference_kernel(ref, ops, N, K):
    fn = _need(ref, "ref_nvfp4_dequant_bf16")
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                   ctypes.c_void_p]
    g = torch.Generator().manual_seed(N * 3 + K)
    packed = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g).cuda()
    # scale bytes over the whole finite ue4m3 range (no NaN code 0x7F / 0xFF)
    sc = torch.randint(0, 0x7F, (N, K // 16), dtype=torch.uint8, generator=g).cuda()
    got = ops.nvfp4_dequant_bf16(packed, sc, 0.37)
    want = torch.zeros_like(got)
    assert fn(_p(packed), _p(sc), 0.37, _p(want), N, K, _stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def _special_rows(M, K, seed):
    """Random rows with values placed exactly on, one float below and one float above every
    e2m1 / e4m3 rounding boundary the quantizers divide by powers of two into, plus zeros of
    both signs, infinities and a NaN."""
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(seed)) * 2
    x[0, :16] = 0.0
    x[0, 3] = -0.0
    x[1, 5] = float("inf")
    x[2, 7] = float("-inf")
    x[3, 9] = float("nan")
    # a group whose largest value is 6 * 2^k has an exact scale; the other values of the group
    # then land exactly on the thresholds after the division
    ties = torch.tensor([6.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, 0.5])
    for r, k in ((4, 0), (5, 3), (6, -2)):
        x[r, 16:32] = ties * 2.0 ** k
    return x.to(torch.bfloat16).cuda()


def test_nvfp4_grouped_special_values_equal_reference_kernel(ref, ops):
    """Ties on every e2m1 threshold (the reference sends them up in magnitude), zeros of both
    signs, infinities and NaN: the bytes of the reference's kernels."""
    K, offs = 256, [0, 5, 5, 12]
    T, E = offs[-1], len(offs) - 1
    xb = _special_rows(T, K, seed=5)
    offs_t = torch.tensor(offs, dtype=torch.int32, device="cuda")
    packed, scales, sf = ops.bf16_to_nvfp4_grouped(xb, offs_t, None)
    wp, wsc = torch.zeros_like(packed), torch.zeros_like(scales)
    assert ref.ref_bf16_to_nvfp4_grouped(_p(xb), _p(wp), _p(wsc), _p(offs_t), _p(sf), T, E, K, None, _stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(packed, wp) and torch.equal(scales, wsc)
    up = _special_rows(T, K, seed=6)
    packed, scales, sf = ops.silu_mul_to_nvfp4_grouped(xb, up, offs_t, None)
    wp, wsc = torch.zeros_like(packed), torch.zeros_like(scales)
    assert ref.ref_silu_mul_to_nvfp4_grouped(_p(xb), _p(up), _p(wp), _p(wsc), _p(offs_t), _p(sf), T, E, K, None,
                                             _stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(packed, wp) and torch.equal(scales, wsc)


@pytest.mark.parametrize("M,K", [(12, 256), (12, 200)])
def test_dynamic_fp8_special_values_equal_reference_kernel(ref, ops, M, K):
    xb = _special_rows(M, K, seed=7)
    out, sc = ops.dynamic_fp8_quant(xb, False)
    want = torch.zeros((M, K), dtype=torch.uint8, device="cuda")
    wsc = torch.zeros_like(sc)
    assert ref.ref_dynamic_fp8_quant(_p(xb), _p(want), _p(wsc), M, K, 0, _stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.uint8), want)
    assert torch.equal(sc.view(torch.int32), wsc.view(torch.int32))   # bit patterns: a NaN scale equals itself
