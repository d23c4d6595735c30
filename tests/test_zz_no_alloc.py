"""GPU test of lsg_gguf_mmvq_noalloc, the entry point for callers that cannot allocate
device memory (fixed memory plans, plug-ins inside another runtime, decode loops that
must stay clear of cudaMalloc).  Its Q8_1 scratch is a device array inside the library.

Collected last on purpose: a run that stops at the first failure has then already
exercised every other test.  It passes alone in a fresh process and after the others."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from layerstormgemmkernels_b200 import quantize as Q
from layerstormgemmkernels_b200.capi import GGUF_TYPES

pytestmark = pytest.mark.gpu


def _call_noalloc(capi, A, W, C, t, N, K, M=None):
    p = capi.GgufMmvqParams(M=A.shape[0] if M is None else M, N=N, K=K, A=A.data_ptr(), B=W.data_ptr(),
                            C=C.data_ptr(), type=t,
                            out_dtype=capi.DTYPE_F32 if C.dtype == torch.float32 else capi.DTYPE_BF16)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return capi.lib.lsg_gguf_mmvq_noalloc(ctypes.byref(p), st)


def test_noalloc_matches_workspace_entry_point_twice_in_a_row():
    from layerstormgemmkernels_b200 import capi, ops
    t = GGUF_TYPES["Q4_K"]
    N = 777
    # two different problems back to back: the second must not see the first's scratch
    for M, K, seed in ((3, 2048, 1), (8, 4096, 2)):
        A = torch.randn(M, K, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16).cuda()
        W = torch.from_numpy(Q.random_gguf_weight("Q4_K", N, K, seed=seed)).cuda()
        want = ops.gguf_mmvq(A, W, t, N, K, out_dtype=torch.float32)   # caller-workspace path
        got = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        capi.check(_call_noalloc(capi, A, W, got, t, N, K))
        torch.cuda.synchronize()
        # same kernels, same inputs: the tolerance of the other parity tests (2e-5 of the
        # output scale) is met with room to spare - the results are in fact identical
        scale = want.abs().max().item()
        assert (got - want).abs().max().item() <= 2e-5 * scale
        assert torch.equal(got, want)
        # and directly against the CPU oracle of the reference's integer path
        bits = A.view(torch.int16).cpu().numpy().view(np.uint16)
        ref = oracle.mmvq(t, oracle.quantize_q8_1(bits), W.cpu().numpy(), K)
        assert np.abs(got.cpu().numpy() - ref).max() <= 2e-5 * np.abs(ref).max()
    assert capi.device_status() == 0


def test_noalloc_bf16_output_other_type_and_empty_shapes():
    """bf16 output (what the reference operator returns), a type with 32-value blocks, and the
    early returns for empty problems (nothing is launched, the output is left alone)."""
    from layerstormgemmkernels_b200 import capi, ops
    for name, M, N, K in (("Q6_K", 2, 320, 1024), ("Q8_0", 5, 130, 512)):
        t = GGUF_TYPES[name]
        A = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).to(torch.bfloat16).cuda()
        W = torch.from_numpy(Q.random_gguf_weight(name, N, K, seed=3)).cuda()
        want = ops.gguf_mmvq(A, W, t, N, K)                               # bf16, caller workspace
        got = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
        capi.check(_call_noalloc(capi, A, W, got, t, N, K))
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        bits = A.view(torch.int16).cpu().numpy().view(np.uint16)
        ref = oracle.mmvq(t, oracle.quantize_q8_1(bits), W.cpu().numpy(), K)
        assert np.abs(got.float().cpu().numpy() - ref).max() <= (2e-5 + 2.0 ** -8) * np.abs(ref).max()
    t = GGUF_TYPES["Q4_K"]
    A = torch.zeros((4, 256), dtype=torch.bfloat16, device="cuda")
    W = torch.zeros((8, 144), dtype=torch.uint8, device="cuda")
    C = torch.full((4, 8), 5.0, dtype=torch.float32, device="cuda")
    assert _call_noalloc(capi, A, W, C, t, 8, 256, M=0) == 0              # M == 0
    assert _call_noalloc(capi, A, W, C, t, 0, 256) == 0                   # N == 0
    torch.cuda.synchronize()
    assert torch.all(C == 5.0)
    assert _call_noalloc(capi, A, W, C, t, 8, 0) != 0                     # K == 0 with rows is an error
    assert capi.device_status() == 0


def test_noalloc_rejects_what_does_not_fit():
    from layerstormgemmkernels_b200 import capi
    t = GGUF_TYPES["Q4_K"]
    M, N, K = 16, 64, 16384          # 16 * 512 * 36 = 294,912 > 147,456
    A = torch.zeros((M, K), dtype=torch.bfloat16, device="cuda")
    W = torch.zeros((N, K // 256 * 144), dtype=torch.uint8, device="cuda")
    C = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    rc = _call_noalloc(capi, A, W, C, t, N, K)
    assert rc == capi.LSG_ERR_WORKSPACE
    assert b"built-in" in capi.lib.lsg_last_error()
    # the largest problem that does fit is accepted
    M = 8
    A = torch.randn((M, K), generator=torch.Generator().manual_seed(0)).to(torch.bfloat16).cuda()
    C = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    capi.check(_call_noalloc(capi, A, W, C, t, N, K))
    torch.cuda.synchronize()
