"""GPU tests of the NVFP4 grouped GEMM.  The reference's arithmetic for this operator lives
in NVIDIA CUTLASS (v4.4.2, sm_120 only; not vendored in the reference), so parity is
anchored on the reference's own tests for the operator (tests/test_kernels.py:273-317,
543-652) and on its Python definition ref_nvfp4_dequant + matmul."""
import numpy as np
import pytest
import torch

import oracle
from layerstormgemmkernels_b200 import quantize as Q
from test_oracle_quant import _decode_grouped

pytestmark = pytest.mark.gpu
UE4M3_ONE = 0x38
TOL = 2e-2        # north-star bound for NVFP4 GEMM outputs


@pytest.fixture(scope="module")
def ops():
    from layerstormgemmkernels_b200 import ops as _ops, capi
    yield _ops
    assert capi.device_status() == 0


def bits_of(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def test_known_answer_all_half(ops):
    """tests/test_kernels.py:273-317: every value 0.5, scales 1 -> K * 0.25."""
    E, M_per, N, K = 4, 128, 128, 128
    T = E * M_per
    A = torch.full((T, K // 2), 0x11, dtype=torch.uint8, device="cuda")
    B = torch.full((E * N, K // 2), 0x11, dtype=torch.uint8, device="cuda")
    sA = torch.full((T * 8,), UE4M3_ONE, dtype=torch.uint8, device="cuda")
    sB = torch.full((E * N * 8,), UE4M3_ONE, dtype=torch.uint8, device="cuda")
    offs = torch.tensor([i * M_per for i in range(E + 1)], dtype=torch.int32, device="cuda")
    ps = torch.tensor([[M_per, N, K]] * E, dtype=torch.int32, device="cuda")
    alphas = torch.ones(E, dtype=torch.float32, device="cuda")
    for dt, td in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
        D = torch.zeros(T, N, dtype=td, device="cuda")
        out = ops.nvfp4_grouped_gemm(A, B, D, sA, sB, alphas, offs, offs, ps, N, K, dt)
        assert out.data_ptr() == D.data_ptr()
        assert torch.equal(D.float(), torch.full((T, N), K * 0.25, device="cuda"))


@pytest.mark.parametrize("N,K,offs,with_is", [
    (128, 256, [0, 5, 5, 133, 163], False),       # reference pairing test: ragged, one empty
    (128, 256, [0, 64, 128], True),               # per-expert input_scales (TRT-LLM scheme)
    (256, 1024, [0, 300, 301, 700], False),
    (384, 512, [0, 0, 17], False),
])
def test_quantizer_to_gemm_pairing(ops, N, K, offs, with_is):
    E, T = len(offs) - 1, offs[-1]
    g = torch.Generator().manual_seed(42 + N)
    scale = 1e-3 if with_is else 1.0
    x = (torch.randn(T, K, generator=g) * scale).to(torch.bfloat16).cuda()
    offs_t = torch.tensor(offs, dtype=torch.int32, device="cuda")
    codes, sbufs, wdeq, alphas = [], [], [], []
    isc = None
    if with_is:
        xf = x.float().cpu().numpy()
        isc = torch.tensor([np.abs(xf[offs[e]:offs[e + 1]]).max() / (448.0 * 6.0) for e in range(E)],
                           dtype=torch.float32, device="cuda")
    for e in range(E):
        w = (torch.randn(N, K, generator=g) * (0.05 if e % 2 else 1.0)).numpy()
        c, sc, s2 = Q.quantize_nvfp4(w)
        codes.append(torch.from_numpy(c).cuda())
        sbufs.append(ops.nvfp4_gemm_preprocess(torch.from_numpy(sc).cuda(), N, K))
        wdeq.append(Q.dequantize_nvfp4(c, sc, 1.0).astype(np.float64))
        alphas.append(float(s2) * (float(isc[e]) if with_is else 1.0))
    A_packed, A_scales, sf = ops.bf16_to_nvfp4_grouped(x, offs_t, isc)
    B = torch.cat(codes, 0)
    sB = torch.cat(sbufs, 0)
    al = torch.tensor(alphas, dtype=torch.float32, device="cuda")
    ps = torch.tensor([[offs[e + 1] - offs[e], N, K] for e in range(E)], dtype=torch.int32, device="cuda")
    D = torch.zeros(T, N, dtype=torch.bfloat16, device="cuda")
    ops.nvfp4_grouped_gemm(A_packed, B, D, A_scales, sB, al, offs_t, sf, ps, N, K, "bf16")
    # oracle: dequantized (bit-exact) activation codes x dequantized weights, float64
    xa = _decode_grouped(A_packed.cpu().numpy(), A_scales.cpu().numpy(), sf.cpu().numpy(), offs, K).astype(np.float64)
    got = D.float().cpu().numpy()
    xf = x.float().cpu().numpy()
    for e in range(E):
        s, t = offs[e], offs[e + 1]
        if s == t:
            continue
        ref = (xa[s:t] @ wdeq[e].T) * np.float64(np.float32(alphas[e]))
        assert np.abs(got[s:t] - ref).max() <= (2.0 ** -8 + 1e-5) * np.abs(ref).max()   # bf16 rounding only
        assert np.abs(got[s:t] - ref).max() <= TOL * np.abs(ref).max()
        # and the reference test's own criterion: cosine > 0.99 vs bf16 activations x dequantized weights
        full = xf[s:t] @ (wdeq[e].T * (alphas[e] / (float(isc[e]) if with_is else 1.0)))
        cos = (full * got[s:t]).sum() / np.sqrt((full * full).sum() * (got[s:t] ** 2).sum())
        assert cos > 0.99


# ---------------------------------------------------------------------------
# Single-problem operators (nvfp4_gemm, bf16_to_nvfp4, nvfp4_gemm_from_bf16)
# ---------------------------------------------------------------------------
def test_single_gemm_known_answer(ops):
    """All values 0.5, scales 1, alpha 2 -> 2 * K * 0.25 (tests/test_kernels.py:244-268 style)."""
    M, N, K = 96, 160, 256
    A = torch.full((M, K // 2), 0x11, dtype=torch.uint8, device="cuda")
    B = torch.full((N, K // 2), 0x11, dtype=torch.uint8, device="cuda")
    sA = torch.full((ops.query_sf_buffer_size_a(M, N, K),), UE4M3_ONE, dtype=torch.uint8, device="cuda")
    sB = torch.full((ops.query_sf_buffer_size_b(M, N, K),), UE4M3_ONE, dtype=torch.uint8, device="cuda")
    for dt, td in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
        D = ops.nvfp4_gemm(A, B, sA, sB, M, N, K, 2.0, dt)
        assert D.dtype == td and tuple(D.shape) == (M, N)
        assert torch.equal(D.float(), torch.full((M, N), 2.0 * K * 0.25, device="cuda"))


@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (37, 256, 512), (300, 96, 1024)])
def test_single_quantizer_equals_grouped_with_one_expert(ops, M, N, K):
    """bf16_to_nvfp4 is the grouped quantizer with one expert and no input scale: same bytes."""
    x = (torch.randn(M, K, generator=torch.Generator().manual_seed(M)) * 0.7).to(torch.bfloat16).cuda()
    codes, sfa = ops.bf16_to_nvfp4(x)
    offs = torch.tensor([0, M], dtype=torch.int32, device="cuda")
    gc, gs, _ = ops.bf16_to_nvfp4_grouped(x, offs, None)
    assert torch.equal(codes, gc)
    n = min(sfa.numel(), gs.numel())
    assert torch.equal(sfa[:n], gs.reshape(-1)[:n])
    # and against the CPU oracle of the grouped quantizer
    oc, osc = oracle.bf16_to_nvfp4_grouped(bits_of(x), np.array([0, M], dtype=np.int32), None)[:2]
    assert np.array_equal(codes.cpu().numpy(), oc)


@pytest.mark.parametrize("M,N,K", [(5, 128, 256), (130, 256, 512)])
def test_single_gemm_from_bf16(ops, M, N, K):
    """bf16 activations -> NVFP4 -> GEMM, against dequantized codes x dequantized weights."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = torch.randn(N, K, generator=g).numpy()
    c, sc, s2 = Q.quantize_nvfp4(w)
    wdeq = Q.dequantize_nvfp4(c, sc, 1.0).astype(np.float64)
    wc = torch.from_numpy(c).cuda()
    out = ops.nvfp4_gemm_from_bf16(x, wc, torch.from_numpy(sc).cuda(), float(s2))
    pre = ops.nvfp4_gemm_preprocess(torch.from_numpy(sc).cuda(), N, K)
    out2 = ops.nvfp4_gemm_from_bf16(x, wc, pre, float(s2))
    assert torch.equal(out, out2)
    codes, sfa = ops.bf16_to_nvfp4(x)
    xa = _decode_grouped(codes.cpu().numpy(), sfa.cpu().numpy(), np.array([0, 0], dtype=np.int32), [0, M], K).astype(np.float64)
    ref = (xa @ wdeq.T) * np.float64(np.float32(s2))
    got = out.float().cpu().numpy()
    assert np.abs(got - ref).max() <= (2.0 ** -8 + 1e-5) * np.abs(ref).max()
    full = x.float().cpu().numpy() @ (wdeq.T * float(s2))
    cos = (full * got).sum() / np.sqrt((full * full).sum() * (got ** 2).sum())
    assert cos > 0.99


@pytest.mark.parametrize("N,K,s2", [(64, 256, 1.0), (130, 512, 0.0371), (1, 16, 3.5)])
def test_nvfp4_dequant_bf16_bit_exact(ops, N, K, s2):
    """(e2m1 * e4m3 scale) * weight_scale_2 in fp32, rounded to bf16: same bits as the formula of
    csrc/smxx/quant/nvfp4_dequant_bf16.h:20-24."""
    rng = np.random.default_rng(N)
    codes = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    sc = rng.integers(0x20, 0x50, size=(N, K // 16), dtype=np.uint8)     # positive, finite e4m3
    out = ops.nvfp4_dequant_bf16(torch.from_numpy(codes).cuda(), torch.from_numpy(sc).cuda(), s2)
    lut = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6], np.float32)
    nib = np.stack([codes & 0xF, codes >> 4], -1).reshape(N, K)
    gs = np.repeat(oracle.e4m3_to_f32(sc).reshape(N, K // 16).astype(np.float32), 16, axis=1)
    val = ((lut[nib] * gs).astype(np.float32) * np.float32(s2)).astype(np.float32)
    exp = torch.from_numpy(val).to(torch.bfloat16)
    assert torch.equal(out.cpu().view(torch.int16), exp.view(torch.int16))
