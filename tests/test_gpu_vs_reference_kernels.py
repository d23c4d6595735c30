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


@pytest.mark.parametrize("M,K", [(1, 4096), (5, 512), (8, 14336), (33, 2048)])
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
