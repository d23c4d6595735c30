"""GPU tests that make the failure paths run without faulting or hanging the GPU: a device
wait that is made to run out reports through the status word, the kernel returns, and the
next call works.  (The reference's kernels never wait; its error convention is the argument
checks of csrc/sm120/gemm/gguf/gguf_grouped_int.cu:933-943, covered by the argument tests.)"""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from layerstormgemmkernels_b200 import quantize as Q
from layerstormgemmkernels_b200.capi import GGUF_TYPES

pytestmark = pytest.mark.gpu


def test_mmvq_wait_that_runs_out_reports_and_the_next_call_works():
    """The producer of the first CTA leaves out one slab of its ring (test hook), so the
    consumers of that slab wait for something nothing will ever publish.  With a limit of
    half a million cycles (a quarter of a millisecond) they give up, record code 1 (data did
    not land) and the kernel returns; the status is read and cleared; the same call without
    the hook then gives the oracle's result."""
    from layerstormgemmkernels_b200 import capi, ops
    lib = capi.lib
    t = GGUF_TYPES["Q4_K"]
    M, N, K = 1, 14336, 4096            # enough rows per CTA for several slabs
    A = torch.randn(M, K, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda()
    Wh = Q.random_gguf_weight("Q4_K", N, K, seed=4)
    W = torch.from_numpy(Wh).cuda()
    assert capi.device_status() == 0
    capi.check(lib.lsg_set_wait_limit_cycles(500000))
    capi.check(lib.lsg_test_mmvq_drop_slab(1))
    try:
        ops.gguf_mmvq(A, W, t, N, K, out_dtype=torch.float32)
        assert capi.device_status() == 1        # synchronizes; the kernel has returned
    finally:
        capi.check(lib.lsg_test_mmvq_drop_slab(-1))
        capi.check(lib.lsg_set_wait_limit_cycles(0))
    assert capi.device_status() == 0
    got = ops.gguf_mmvq(A, W, t, N, K, out_dtype=torch.float32).cpu().numpy()
    bits = A.view(torch.int16).cpu().numpy().view(np.uint16)
    ref = oracle.mmvq(t, oracle.quantize_q8_1(bits), Wh, K)
    assert np.abs(got - ref).max() <= 2e-5 * np.abs(ref).max()
    assert capi.device_status() == 0


def test_wait_limit_setter_rejects_negative_values():
    from layerstormgemmkernels_b200 import capi
    with pytest.raises(ValueError):
        capi.check(capi.lib.lsg_set_wait_limit_cycles(-5))
    capi.check(capi.lib.lsg_set_wait_limit_cycles(0))
