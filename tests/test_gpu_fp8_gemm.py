"""GPU tests of the FP8 (e4m3) block-scaled GEMM family and the weight quantizer.  The
reference's GEMM arithmetic for these operators lives in NVIDIA CUTLASS (sm_120 only, not
vendored in the reference), so parity is anchored on the operand contract of
csrc/sm120/gemm/fp8/fp8_gemm.h:18-44 restated in float64 here, on the reference's weight
quantizer (csrc/smxx/quant/weight_fp8_quant.cu:51-138) restated in numpy, and on the cases of
tests/test_kernels.py that pair the quantizers with the GEMM."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
TOL = 1e-3


@pytest.fixture(scope="module")
def ops():
    from layerstormgemmkernels_b200 import ops as _ops, capi
    yield _ops
    assert capi.device_status() == 0


def raw(t):
    return t.view(torch.uint8).cpu().numpy()


@pytest.mark.parametrize("N,K", [(128, 128), (300, 384), (256, 1040), (1, 16)])
def test_weight_fp8_quant_bit_exact(ops, N, K):
    w = (torch.randn(N, K, generator=torch.Generator().manual_seed(N + K)) * 0.3).to(torch.bfloat16)
    if N > 128:
        w[128:256, :min(K, 128)] = 0            # an all-zero tile: scale 1
    q, s = ops.weight_fp8_quant(w.cuda())
    assert q.dtype == torch.float8_e4m3fn and tuple(s.shape) == ((N + 127) // 128, (K + 127) // 128)
    exp_q, exp_s = oracle.weight_fp8_quant(w.float().numpy())
    assert np.array_equal(s.cpu().numpy(), exp_s)
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), exp_q)


@pytest.mark.parametrize("M,N,K", [(1, 256, 256), (5, 200, 384), (130, 384, 1024), (64, 128, 2048)])
def test_fp8_gemm_quantizer_pairing(ops, M, N, K):
    g = torch.Generator().manual_seed(M * 7 + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    a8, sa = ops.dynamic_fp8_quant(x, True)        # scales [KB, M] = M-major
    b8, sb = ops.weight_fp8_quant(w)               # scales [NB, KB] = K-major
    ref = oracle.fp8_gemm(raw(a8), sa.cpu().numpy(), raw(b8), sb.cpu().numpy(), M, N, K)
    for dt, td in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
        out = ops.fp8_gemm(a8, b8, sa, sb, M, N, K, dt)
        assert out.dtype == td and tuple(out.shape) == (M, N)
        slack = 2.0 ** -8 if td == torch.bfloat16 else 2.0 ** -11
        assert np.abs(out.float().cpu().numpy() - ref).max() <= (TOL + slack) * np.abs(ref).max()
    # and close to the unquantized product, as the reference's tests check (cosine)
    full = x.float().cpu().numpy().astype(np.float64) @ w.float().cpu().numpy().astype(np.float64).T
    got = out.float().cpu().numpy()
    assert (full * got).sum() / np.sqrt((full * full).sum() * (got * got).sum()) > 0.99


def test_fp8_grouped_gemm_ragged_experts(ops):
    N, K = 256, 512
    offs = [0, 40, 40, 170, 173]
    E, T = len(offs) - 1, offs[-1]
    g = torch.Generator().manual_seed(9)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).cuda()
    ws = [(torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda() for _ in range(E)]
    a8 = torch.empty((T, K), dtype=torch.float8_e4m3fn, device="cuda")
    KB = K // 128
    sa = torch.zeros((T * KB,), dtype=torch.float32, device="cuda")
    refs = []
    b8s, sbs = [], []
    for e in range(E):
        q, s = ops.weight_fp8_quant(ws[e])
        b8s.append(q)
        sbs.append(s.reshape(-1))
    for e in range(E):
        s0, s1 = offs[e], offs[e + 1]
        if s0 == s1:
            refs.append(None)
            continue
        qa, sc = ops.dynamic_fp8_quant(x[s0:s1].contiguous(), True)     # M-major inside the expert
        a8[s0:s1] = qa
        sa[s0 * KB:s1 * KB] = sc.reshape(-1)
        refs.append(oracle.fp8_gemm(raw(qa), sc.cpu().numpy(), raw(b8s[e]), sbs[e].cpu().numpy(), s1 - s0, N, K))
    B = torch.cat([q.view(torch.uint8) for q in b8s], 0).view(torch.float8_e4m3fn)
    sB = torch.cat(sbs, 0)
    offs_t = torch.tensor(offs, dtype=torch.int32, device="cuda")
    ps = torch.tensor([[offs[e + 1] - offs[e], N, K] for e in range(E)], dtype=torch.int32, device="cuda")
    D = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    out = ops.fp8_grouped_gemm(a8, B, D, sa, sB, offs_t, ps, N, K, "bf16")
    assert out.data_ptr() == D.data_ptr()
    got = D.float().cpu().numpy()
    for e in range(E):
        if refs[e] is None:
            continue
        s0, s1 = offs[e], offs[e + 1]
        assert np.abs(got[s0:s1] - refs[e]).max() <= (TOL + 2.0 ** -8) * np.abs(refs[e]).max()


@pytest.mark.parametrize("M", [1, 2, 3, 4])
@pytest.mark.parametrize("N,K", [(200, 384), (4096, 7168)])
def test_fp8_small_batch_matvec(ops, M, N, K):
    """M <= 4 takes the streaming mat-vec kernel (role of fp8_blockscaled_gemv.cu:54-145):
    fp32 products and scaling, so it agrees with the float64 contract far inside the bound."""
    g = torch.Generator().manual_seed(N + M)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    a8, sa = ops.dynamic_fp8_quant(x, True)
    b8, sb = ops.weight_fp8_quant(w)
    ref = oracle.fp8_gemm(raw(a8), sa.cpu().numpy(), raw(b8), sb.cpu().numpy(), M, N, K)
    out = ops.fp8_gemm(a8, b8, sa, sb, M, N, K, "bf16").float().cpu().numpy()
    assert np.abs(out - ref).max() <= (1e-5 + 2.0 ** -8) * np.abs(ref).max()
