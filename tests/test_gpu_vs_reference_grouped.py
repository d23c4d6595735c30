"""GPU tests against the reference's OWN grouped (MoE) kernels, routing-metadata kernels,
mma.sync prefill GEMM and FP8 weight quantizer, compiled for sm_100a from the reference
checkout into oracle/_ref/libref_grouped.so (`make -C oracle ref`).  Skipped when that
library has not been built.  Reference: csrc/sm120/gemm/gguf/gguf_grouped_int.cu:46-66,
156-187, 925-995; mmq_mma/mmq_mma_dispatch.cu:52-91; csrc/smxx/quant/weight_fp8_quant.cu."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from layerstormgemmkernels_b200 import quantize as Q
from layerstormgemmkernels_b200.capi import GGUF_TYPES

pytestmark = pytest.mark.gpu
T = GGUF_TYPES
REF_TYPES = ["Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "Q8_0", "MXFP4"]


@pytest.fixture(scope="module")
def ref():
    lib = oracle.ref_grouped_lib()
    if lib is None:
        pytest.skip("oracle/_ref/libref_grouped.so not built")
    return lib


@pytest.fixture(scope="module")
def ops():
    from layerstormgemmkernels_b200 import ops as _ops, capi
    yield _ops
    assert capi.device_status() == 0


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


OFFSETS = [[0, 5, 5, 133, 163], [0, 0, 0, 7], [0, 64, 128, 192, 256], [0, 300, 301, 700, 700, 1000], [0, 1]]


@pytest.mark.parametrize("offs", OFFSETS)
@pytest.mark.parametrize("tile_m", [64, 128])
def test_tile_map_bit_exact_vs_reference_kernel(ref, ops, offs, tile_m):
    E, total = len(offs) - 1, offs[-1]
    o = torch.tensor(offs, dtype=torch.int32, device="cuda")
    t_max = (total + tile_m - 1) // tile_m + E
    want_e = torch.full((t_max,), 99, dtype=torch.int32, device="cuda")
    want_m = torch.full((t_max,), 99, dtype=torch.int32, device="cuda")
    assert ref.ref_build_mmq_tile_map(_p(o), E, tile_m, t_max, _p(want_e), _p(want_m), _stream()) == 0
    got_e, got_m = ops.build_mmq_tile_map(o, tile_m, t_max)
    torch.cuda.synchronize()
    assert torch.equal(got_e, want_e) and torch.equal(got_m, want_m)


@pytest.mark.parametrize("offs", OFFSETS)
def test_active_expert_list_bit_exact_vs_reference_kernel(ref, ops, offs):
    E, total = len(offs) - 1, offs[-1]
    o = torch.tensor(offs, dtype=torch.int32, device="cuda")
    cap = min(E, total)
    want = torch.full((max(cap, 1),), 99, dtype=torch.int32, device="cuda")
    assert ref.ref_build_active_expert_list(_p(o), E, cap, _p(want), _stream()) == 0
    got = ops.build_active_expert_list(o, cap)
    torch.cuda.synchronize()
    assert torch.equal(got[:cap], want[:cap])


def _grouped_case(name, offs, N, K, seed):
    E, total = len(offs) - 1, offs[-1]
    g = torch.Generator().manual_seed(seed)
    A = (torch.randn(total, K, generator=g) * 0.4).to(torch.bfloat16).cuda()
    Ws = [torch.from_numpy(Q.random_gguf_weight(name, N, K, seed=seed + e)).cuda() for e in range(E)]
    bp = torch.tensor([w.data_ptr() for w in Ws], dtype=torch.int64, device="cuda")
    o = torch.tensor(offs, dtype=torch.int32, device="cuda")
    return A, Ws, bp, o


@pytest.mark.parametrize("name", REF_TYPES)
@pytest.mark.parametrize("force,offs", [(1, [0, 3, 3, 8, 12]), (2, [0, 70, 70, 200, 333])])
def test_grouped_gemm_vs_reference_kernels(ref, ops, name, force, offs):
    """Int strategy, mmvq (force 1) and mmq (force 2) sub-paths: this library's grouped GEMM
    against the reference's device-routed kernels on the same inputs.  Both compute the same
    integer dots; the tensor-core route here rounds its operands to fp16 (bound 1e-3)."""
    N, K = 256, 512
    E, total = len(offs) - 1, offs[-1]
    A, Ws, bp, o = _grouped_case(name, offs, N, K, seed=11)
    ws_bytes = int(ref.ref_gguf_grouped_gemm_workspace_bytes(total, K, E))
    ws = torch.empty((max(ws_bytes, 256),), dtype=torch.uint8, device="cuda")
    want = torch.zeros((total, N), dtype=torch.bfloat16, device="cuda")
    rc = ref.ref_gguf_grouped_gemm(T[name], 1, E, N, K, _p(A), _p(want), _p(o), _p(bp), total, _p(ws),
                                   ctypes.c_size_t(ws_bytes), force, _stream())
    assert rc == 0
    got = ops.gguf_grouped_gemm(A, o, bp, T[name], 1, N, K, force=force, out_dtype=torch.float32)
    torch.cuda.synchronize()
    w, g = want.float().cpu().numpy(), got.cpu().numpy()
    rows = np.concatenate([np.arange(offs[e], offs[e + 1]) for e in range(E)])
    err = np.abs(g[rows] - w[rows]).max() / np.abs(w[rows]).max()
    assert err <= 1e-3 + 2.0 ** -8, (name, force, err)      # the reference output is bf16


@pytest.mark.parametrize("name", REF_TYPES)
def test_prefill_gemm_vs_reference_mma_kernel(ref, ops, name):
    M, N, K = 200, 384, 1024
    A = (torch.randn(M, K, generator=torch.Generator().manual_seed(5)) * 0.4).to(torch.bfloat16).cuda()
    W = torch.from_numpy(Q.random_gguf_weight(name, N, K, seed=9)).cuda()
    ws = torch.empty((M * (K // 32) * 36 + 256,), dtype=torch.uint8, device="cuda")
    want = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    assert ref.ref_gguf_mmq_mma(M, N, K, _p(A), _p(W), _p(want), T[name], _p(ws), _stream()) == 0
    got = ops.gguf_mmq(A, W, T[name], N, K, out_dtype=torch.float32)
    torch.cuda.synchronize()
    w, g = want.float().cpu().numpy(), got.cpu().numpy()
    assert np.abs(g - w).max() <= (1e-3 + 2.0 ** -8) * np.abs(w).max()


@pytest.mark.parametrize("N,K", [(256, 384), (200, 130), (128, 128)])
def test_weight_fp8_quant_bit_exact_vs_reference_kernel(ref, ops, N, K):
    w = (torch.randn(N, K, generator=torch.Generator().manual_seed(N)) * 0.1).to(torch.bfloat16).cuda()
    nb, kb = (N + 127) // 128, (K + 127) // 128
    want_q = torch.zeros((N, K), dtype=torch.uint8, device="cuda")
    want_s = torch.zeros((kb * nb,), dtype=torch.float32, device="cuda")
    assert ref.ref_weight_fp8_quant(_p(w), _p(want_q), _p(want_s), N, K, _stream()) == 0
    q, s = ops.weight_fp8_quant(w)
    torch.cuda.synchronize()
    assert torch.equal(q.view(torch.uint8), want_q)
    assert torch.equal(s.reshape(-1), want_s)
