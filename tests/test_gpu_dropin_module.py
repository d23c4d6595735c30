"""GPU tests through the drop-in PyTorch extension `sm120_gemm_kernels` (the reference's
module name), written the way the reference's own tests call it
(tests/test_gguf_mmvq.py, tests/test_gguf_grouped_gemm.py, tests/test_kernels.py)."""
import os
import sys

import numpy as np
import pytest
import torch

from layerstormgemmkernels_b200 import quantize as Q

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GGUF_T = {"Q2_K": 0, "Q3_K": 1, "Q4_K": 2, "Q5_K": 3, "Q6_K": 4, "Q8_0": 5, "MXFP4": 6}
F_AUTO, F_MMVQ, F_MMQ, F_HOSTLOOP = 0, 1, 2, 3
S_DEQUANT, S_INT = 0, 1


@pytest.fixture(scope="module")
def GK():
    if not os.path.exists(os.path.join(ROOT, "sm120_gemm_kernels.so")):
        pytest.skip("sm120_gemm_kernels.so not built (python -m layerstormgemmkernels_b200.torch_ext.build_ext)")
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    import sm120_gemm_kernels
    return sm120_gemm_kernels


def cosine(a, b):
    a, b = a.float().flatten(), b.float().flatten()
    return torch.nn.functional.cosine_similarity(a.unsqueeze(0), b.unsqueeze(0)).item()


@pytest.mark.parametrize("name", list(GGUF_T))
@pytest.mark.parametrize("M", [1, 3, 8, 12, 17])
def test_mmvq_vs_goldens(GK, name, M):
    """tests/test_gguf_mmvq.py:55-72."""
    torch.manual_seed(0)
    N, K = 320, 512
    A = (torch.randn(M, K) * 0.4).to(torch.bfloat16).cuda()
    W = torch.from_numpy(Q.random_gguf_weight(name, N, K, seed=42)).cuda()
    out = GK.gguf_mmvq(A, W, GGUF_T[name], N, K)
    off = torch.tensor([0, M], dtype=torch.int32, device="cuda")
    bptr = torch.tensor([W.data_ptr()], dtype=torch.int64, device="cuda")
    dq = GK.gguf_grouped_gemm(A, off, bptr, GGUF_T[name], S_DEQUANT, N, K, F_HOSTLOOP)
    gi = GK.gguf_grouped_gemm(A, off, bptr, GGUF_T[name], S_INT, N, K, F_MMVQ)
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (M, N)
    assert cosine(dq, out) >= 0.999
    assert cosine(gi, out) >= 0.9995
    assert torch.equal(gi, out)     # same integer math, same reduction order


def test_grouped_dists_and_graph(GK):
    """tests/test_gguf_grouped_gemm.py:129-159, 227-261 for Q4_K."""
    E, K, N = 6, 256, 256
    for counts in ([1 + (e % 8) for e in range(E)], [64 + 40 * (e % 4) for e in range(E)],
                   [0 if e % 3 == 0 else (1 + (e % 7)) for e in range(E)]):
        offs = np.zeros(E + 1, np.int32)
        offs[1:] = np.cumsum(counts)
        A = (torch.randn(int(offs[-1]), K, generator=torch.Generator().manual_seed(100)) * 0.4).to(torch.bfloat16).cuda()
        ws = [torch.from_numpy(Q.random_gguf_weight("Q4_K", N, K, 101 + e)).cuda() for e in range(E)]
        bp = torch.tensor([w.data_ptr() for w in ws], dtype=torch.int64, device="cuda")
        off = torch.from_numpy(offs).cuda()
        golden = GK.gguf_grouped_gemm(A, off, bp, 2, S_DEQUANT, N, K, F_HOSTLOOP)
        host_int = GK.gguf_grouped_gemm(A, off, bp, 2, S_INT, N, K, F_HOSTLOOP)
        live = torch.cat([torch.arange(offs[e], offs[e + 1]) for e in range(E) if counts[e] > 0]).cuda()
        for force in (F_AUTO, F_MMVQ, F_MMQ):
            out = GK.gguf_grouped_gemm(A, off, bp, 2, S_INT, N, K, force)
            assert cosine(golden[live], out[live]) >= 0.999
            assert cosine(host_int[live], out[live]) >= 0.9995
    g = torch.cuda.CUDAGraph()
    eager = GK.gguf_grouped_gemm(A, off, bp, 2, S_INT, N, K)
    torch.cuda.synchronize()
    with torch.cuda.graph(g):
        cap = GK.gguf_grouped_gemm(A, off, bp, 2, S_INT, N, K)
    cap.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(eager[live], cap[live])


def test_fp8_quant_roundtrip(GK):
    """tests/test_kernels.py:147-164."""
    x = torch.randn(32, 1024).to(torch.bfloat16).cuda()
    out, scales = GK.dynamic_fp8_quant(x)
    assert out.dtype == torch.float8_e4m3fn and tuple(scales.shape) == (32, 8)
    deq = out.float().view(32, 8, 128) * scales.view(32, 8, 1)
    assert cosine(x, deq.view(32, 1024)) > 0.999
    out2, sc2 = GK.dynamic_fp8_quant(x, m_major_scales=True)
    assert tuple(sc2.shape) == (8, 32) and torch.equal(sc2.t().contiguous(), scales)


def test_nvfp4_known_answer_and_fused_identity(GK):
    """tests/test_kernels.py:273-317 and 667-731 (against this library's unfused sequence)."""
    E, M_per, N, K = 4, 128, 128, 128
    T = E * M_per
    A = torch.full((T, K // 2), 0x11, dtype=torch.uint8, device="cuda")
    B = torch.full((E * N, K // 2), 0x11, dtype=torch.uint8, device="cuda")
    sA = torch.full((T, 8), 0x38, dtype=torch.uint8, device="cuda")
    sB = torch.full((E * N, 8), 0x38, dtype=torch.uint8, device="cuda")
    offs = torch.tensor([i * M_per for i in range(E + 1)], dtype=torch.int32, device="cuda")
    ps = torch.tensor([[M_per, N, K]] * E, dtype=torch.int32, device="cuda")
    D = torch.zeros(T, N, dtype=torch.bfloat16, device="cuda")
    GK.nvfp4_grouped_gemm(A, B, D, sA, sB, torch.ones(E, device="cuda"), offs, offs, ps, N, K, "bf16")
    assert torch.equal(D.float(), torch.full((T, N), K * 0.25, device="cuda"))
    gate = torch.randn(T, 256).to(torch.bfloat16).cuda()
    up = torch.randn(T, 256).to(torch.bfloat16).cuda()
    p, s, sf = GK.silu_mul_to_nvfp4_grouped(gate, up, offs)
    assert tuple(p.shape) == (T, 128) and s.numel() == T * 16 and sf.tolist() == offs.tolist()
    with pytest.raises(ValueError):          # K must be a multiple of 16
        GK.fp8_gemm(A, A, A, A, 1, 1, 1, "bf16")


def test_errors_raise_like_the_reference(GK):
    A = torch.zeros(1, 100, dtype=torch.bfloat16, device="cuda")
    W = torch.zeros(8, 144, dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError):          # std::invalid_argument from the launcher
        GK.gguf_mmvq(A, W, 2, 8, 100)
    with pytest.raises(RuntimeError):        # TORCH_CHECK
        GK.gguf_mmvq(A.float(), W, 2, 8, 100)


def test_legacy_q4k_gemm_operators(GK):
    """q4k_dequant_gemm / q4k_cutlass_gemm (tests/test_kernels.py:736-820 of the reference):
    x_bf16 @ dequant(W_q4k).T -> bf16, checked against the fp32 dequant-then-matmul oracle."""
    import oracle
    from layerstormgemmkernels_b200 import quantize as Q
    from layerstormgemmkernels_b200.capi import GGUF_TYPES
    M, N, K = 40, 384, 512
    x = (torch.randn(M, K, generator=torch.Generator().manual_seed(5)) * 0.5).to(torch.bfloat16).cuda()
    W = Q.quantize_q4_k((np.random.default_rng(5).standard_normal((N, K)) * 0.02).astype(np.float32))
    Wd = torch.from_numpy(W).cuda()
    ref = oracle.dequant_gemm(GGUF_TYPES["Q4_K"], x.view(torch.int16).cpu().numpy().view(np.uint16), W, K)
    for fn in (GK.q4k_dequant_gemm, GK.q4k_cutlass_gemm):
        out = fn(x, Wd)
        assert out.dtype == torch.bfloat16 and tuple(out.shape) == (M, N)
        assert np.abs(out.float().cpu().numpy() - ref).max() <= (1e-3 + 2.0 ** -8) * np.abs(ref).max()
    with pytest.raises(RuntimeError):
        GK.q4k_dequant_gemm(x[:, :500].contiguous(), Wd)
