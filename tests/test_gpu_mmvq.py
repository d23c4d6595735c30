"""GPU parity tests for the GGUF decode path, through the C ABI, against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

import oracle
from layerstormgemmkernels_b200 import quantize as Q
from layerstormgemmkernels_b200.capi import GGUF_TYPES, BLOCK_BYTES, BLOCK_VALUES

pytestmark = pytest.mark.gpu
T = GGUF_TYPES

# GEMM parity bound of the north star: max |y - ref| / max |ref| <= 1e-3.  The fp32
# accumulator output is held to 2e-5 (it only differs from the oracle by summation order).
TOL_BF16 = 2.0 ** -8 + 1e-4  # bf16 rounding alone is up to half an ulp = 2^-8 relative
TOL_F32 = 2e-5


@pytest.fixture(scope="module")
def ops():
    from layerstormgemmkernels_b200 import ops as _ops, capi
    assert torch.cuda.is_available()
    yield _ops
    assert capi.device_status() == 0, "a kernel reported a timed-out device-side wait"


def bf16_bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def rel_err(got, ref):
    return np.abs(got.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30)


@pytest.mark.parametrize("M,K", [(1, 32), (1, 4096), (3, 512), (8, 14336), (17, 256), (64, 2048), (611, 4096)])
def test_q8_1_quantizer_bit_exact(ops, M, K):
    g = torch.Generator().manual_seed(M * 1000 + K)
    x = torch.randn(M, K, generator=g)
    x[0, :32] = 0.0                       # all-zero block -> d = 0, q = 0
    if K >= 64:
        x[-1, 32:64] *= 1e-3              # small block
        x[-1, 40] = 3e4                   # large outlier
    xb = x.to(torch.bfloat16).cuda()
    got = ops.quantize_q8_1(xb).cpu().numpy()
    ref = oracle.quantize_q8_1(bf16_bits(xb))
    np.testing.assert_array_equal(got, ref)


@pytest.mark.parametrize("name", list(T))
def test_dequant_blocks_match_oracle(ops, name):
    t = T[name]
    K = 512
    W = Q.random_gguf_weight(name, 33, K, seed=21)
    got = ops.gguf_dequant(torch.from_numpy(W).cuda(), t).cpu().numpy()
    ref = oracle.dequant(t, W)
    # same fp32 operations; fused multiply-add contraction may differ in the last bit
    np.testing.assert_allclose(got, ref, rtol=3e-7, atol=1e-9)


@pytest.mark.parametrize("name", list(T))
@pytest.mark.parametrize("M", [1, 2, 3, 4, 8, 12, 17])
def test_mmvq_matches_oracle_small(ops, name, M):
    """The reference's own test shape (tests/test_gguf_mmvq.py:55-72): N=320, K=512."""
    t = T[name]
    N, K = 320, 512
    g = torch.Generator().manual_seed(M)
    A = (torch.randn(M, K, generator=g) * 0.4).to(torch.bfloat16).cuda()
    W = Q.random_gguf_weight(name, N, K, seed=42)
    Wd = torch.from_numpy(W).cuda()
    xq = oracle.quantize_q8_1(bf16_bits(A))
    ref = oracle.mmvq(t, xq, W, K)
    got32 = ops.gguf_mmvq(A, Wd, t, N, K, out_dtype=torch.float32).cpu().numpy()
    assert rel_err(got32, ref) <= TOL_F32
    got16 = ops.gguf_mmvq(A, Wd, t, N, K).float().cpu().numpy()
    assert rel_err(got16, ref) <= TOL_BF16
    # bf16 output must be exactly the rounding of the fp32 accumulator
    np.testing.assert_array_equal(
        got16, torch.from_numpy(got32).to(torch.bfloat16).float().numpy())


@pytest.mark.parametrize("name,N,K,M", [
    ("Q4_K", 1536, 2048, 1), ("Q8_0", 1536, 2048, 1),     # reference decode shape
    ("Q4_K", 1024, 4096, 1), ("Q4_K", 1024, 4096, 8),     # k/v projection
    ("Q6_K", 1024, 4096, 2), ("Q6_K", 1000, 4096, 4),     # N not a multiple of anything
    ("Q4_K", 301, 14336, 1), ("Q4_K", 301, 14336, 8),     # long K: smem activations
    ("Q6_K", 150, 14336, 5), ("Q4_0", 777, 4096, 1),
    ("Q8_0", 600, 4096, 3), ("MXFP4", 513, 2048, 2),
    ("Q2_K", 300, 768, 1), ("Q3_K", 300, 768, 7), ("Q5_K", 129, 768, 4),  # K=768: 12 chunks
    ("Q4_K", 5, 256, 1), ("Q8_0", 3, 32, 1), ("MXFP4", 7, 32, 2), ("Q4_0", 1, 96, 9),
])
def test_mmvq_matches_oracle_shapes(ops, name, N, K, M):
    t = T[name]
    g = torch.Generator().manual_seed(N + K + M)
    A = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    W = Q.random_gguf_weight(name, N, K, seed=N)
    Wd = torch.from_numpy(W).cuda()
    ref = oracle.mmvq(t, oracle.quantize_q8_1(bf16_bits(A)), W, K)
    got = ops.gguf_mmvq(A, Wd, t, N, K, out_dtype=torch.float32).cpu().numpy()
    assert rel_err(got, ref) <= TOL_F32


@pytest.mark.parametrize("name", ["Q4_K", "Q6_K", "Q8_0", "Q4_0"])
def test_mmvq_real_quantized_weights_vs_dequant_golden(ops, name, golden_dir):
    """Weights quantized from N(0, 0.02): integer path vs lossless-activation golden
    (cosine >= 0.999 is the reference's own acceptance bound, test_gguf_mmvq.py:65-68)."""
    t = T[name]
    N, K, M = 256, 1024, 4
    rng = np.random.default_rng(1)
    W = Q.QUANTIZERS[name]((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    A = torch.randn(M, K, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).cuda()
    Wd = torch.from_numpy(W).cuda()
    out = ops.gguf_mmvq(A, Wd, t, N, K, out_dtype=torch.float32).cpu().numpy()
    gold = ops.gguf_dequant_gemm(A, Wd, t, N, K, out_dtype=torch.float32).cpu().numpy()
    gold_cpu = oracle.dequant_gemm(t, bf16_bits(A), W, K)
    assert rel_err(gold, gold_cpu) <= TOL_F32
    cos = (out * gold).sum() / np.sqrt((out * out).sum() * (gold * gold).sum())
    assert cos >= 0.999


def test_mmvq_q4k_golden_fixture(ops, golden_dir):
    """Weights packed by the reference's own quantize_to_q4k (committed fixture)."""
    z = np.load(os.path.join(golden_dir, "q4k_reference.npz"))
    W = z["packed"]
    A = torch.from_numpy(z["x_bf16"].view(np.int16)).view(torch.bfloat16).cuda()
    Wd = torch.from_numpy(W).cuda()
    N, K = W.shape[0], 512
    gold = ops.gguf_dequant_gemm(A, Wd, T["Q4_K"], N, K, out_dtype=torch.float32).cpu().numpy()
    assert rel_err(gold, z["gemm"].astype(np.float64)) <= TOL_F32
    ref = oracle.mmvq(T["Q4_K"], oracle.quantize_q8_1(z["x_bf16"]), W, K)
    got = ops.gguf_mmvq(A, Wd, T["Q4_K"], N, K, out_dtype=torch.float32).cpu().numpy()
    assert rel_err(got, ref) <= TOL_F32


def test_mmvq_bit_deterministic(ops):
    """tests/test_gguf_mmvq.py:91-103."""
    N, K = 640, 1024
    A = (torch.randn(3, K, generator=torch.Generator().manual_seed(2)) * 0.4).to(torch.bfloat16).cuda()
    W = torch.from_numpy(Q.random_gguf_weight("Q8_0", N, K, seed=9)).cuda()
    ref = ops.gguf_mmvq(A, W, T["Q8_0"], N, K)
    for _ in range(5):
        assert torch.equal(ref, ops.gguf_mmvq(A, W, T["Q8_0"], N, K))


@pytest.mark.parametrize("name,M,pinned", [("Q4_K", 1, True), ("Q6_K", 3, True), ("Q8_0", 2, False),
                                            ("Q4_K", 12, True)])
def test_mmvq_host_buffers_equal_device_call(ops, name, M, pinned):
    """lsg_gguf_mmvq_host (activations and result in host memory) returns the bits of the
    device-memory call, for page-locked and pageable buffers, bf16 and f32 results."""
    N, K = 768, 2048
    A = (torch.randn(M, K, generator=torch.Generator().manual_seed(5)) * 0.4).to(torch.bfloat16)
    W = torch.from_numpy(Q.random_gguf_weight(name, N, K, seed=13)).cuda()
    for dt in (torch.bfloat16, torch.float32):
        ref = ops.gguf_mmvq(A.cuda(), W, T[name], N, K, out_dtype=dt).cpu()
        a = A.pin_memory() if pinned else A
        out = torch.zeros((M, N), dtype=dt)
        if pinned:
            out = out.pin_memory()
        got = ops.gguf_mmvq_host(a, W, T[name], N, K, out=out)
        torch.cuda.synchronize()
        assert got is out and torch.equal(got, ref)
    with pytest.raises(RuntimeError):
        ops.gguf_mmvq_host(A, W, T[name], N, K, workspace=torch.empty(16, dtype=torch.uint8, device="cuda"))


def test_mmvq_host_batch_shares_quantized_activations(ops):
    """lsg_gguf_mmvq_host_batch: seven projections of a decoder layer's shapes (scaled down),
    three distinct activations, equal to the per-projection device calls bit for bit; a second
    run() picks up new activation contents."""
    H, I, KV = 1024, 2560, 256
    shapes = [(H, H), (KV, H), (KV, H), (H, H), (I, H), (I, H), (H, I)]
    g = torch.Generator().manual_seed(21)
    xs = [(torch.randn(2, K, generator=g) * 0.4).to(torch.bfloat16).pin_memory() for K in (H, H, I)]
    which = [0, 0, 0, 1, 0, 0, 2]
    Ws = [torch.from_numpy(Q.random_gguf_weight("Q4_K", N, K, seed=30 + i)).cuda()
          for i, (N, K) in enumerate(shapes)]
    items = [(xs[w], W, T["Q4_K"], N, K, None) for w, W, (N, K) in zip(which, Ws, shapes)]
    batch = ops.HostMmvqBatch(items)
    for rnd in range(4):
        if rnd == 2:
            batch.capture()     # the last two rounds replay a CUDA graph of the batch
        outs = batch.run()
        torch.cuda.synchronize()
        for w, W, (N, K), out in zip(which, Ws, shapes, outs):
            assert torch.equal(out, ops.gguf_mmvq(xs[w].cuda(), W, T["Q4_K"], N, K).cpu())
        for x in xs:
            x.mul_(-0.5)
    with pytest.raises(RuntimeError):
        ops.HostMmvqBatch(items, workspace=torch.empty(16, dtype=torch.uint8, device="cuda"))


def test_mmvq_host_batch_chained_projection_reads_the_earlier_result(ops):
    """A projection whose input is the host buffer an earlier projection of the same batch writes:
    the batch must not quantize that input up front with the others."""
    from layerstormgemmkernels_b200 import capi
    import ctypes
    K0, N0, N1 = 512, 256, 96          # y0 = x W0^T (bf16 [1, 256]), y1 = y0 W1^T
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(1, K0, generator=g) * 0.5).to(torch.bfloat16).pin_memory()
    x2 = (torch.randn(1, K0, generator=g) * 0.5).to(torch.bfloat16).pin_memory()
    W0 = torch.from_numpy(Q.random_gguf_weight("Q4_K", N0, K0, seed=1)).cuda()
    W1 = torch.from_numpy(Q.random_gguf_weight("Q4_K", N1, N0, seed=2)).cuda()
    W2 = torch.from_numpy(Q.random_gguf_weight("Q4_K", N1, K0, seed=3)).cuda()
    y0 = torch.zeros((1, N0), dtype=torch.bfloat16).pin_memory()
    y1 = torch.zeros((1, N1), dtype=torch.bfloat16).pin_memory()
    y2 = torch.zeros((1, N1), dtype=torch.bfloat16).pin_memory()
    arr = (capi.GgufMmvqParams * 3)()
    t = T["Q4_K"]
    arr[0] = capi.GgufMmvqParams(M=1, N=N0, K=K0, A=x.data_ptr(), B=W0.data_ptr(), C=y0.data_ptr(), type=t, out_dtype=capi.DTYPE_BF16)
    arr[1] = capi.GgufMmvqParams(M=1, N=N1, K=N0, A=y0.data_ptr(), B=W1.data_ptr(), C=y1.data_ptr(), type=t, out_dtype=capi.DTYPE_BF16)
    arr[2] = capi.GgufMmvqParams(M=1, N=N1, K=K0, A=x2.data_ptr(), B=W2.data_ptr(), C=y2.data_ptr(), type=t, out_dtype=capi.DTYPE_BF16)
    need = capi.lib.lsg_gguf_mmvq_host_batch_workspace_bytes(arr, 3)
    ws = torch.empty((need,), dtype=torch.uint8, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    capi.check(capi.lib.lsg_gguf_mmvq_host_batch(arr, 3, ctypes.c_void_p(ws.data_ptr()), need, st))
    torch.cuda.synchronize()
    r0 = ops.gguf_mmvq(x.cuda(), W0, t, N0, K0)
    assert torch.equal(y0, r0.cpu())
    assert torch.equal(y1, ops.gguf_mmvq(r0, W1, t, N1, N0).cpu())
    assert torch.equal(y2, ops.gguf_mmvq(x2.cuda(), W2, t, N1, K0).cpu())


@pytest.mark.parametrize("name,M", [("Q4_K", 1), ("Q4_K", 3), ("Q6_K", 2)])
def test_mmvq_batch_distinct_inputs_share_a_launch(ops, name, M):
    """A decoder layer's seven projections (scaled down) with their four distinct inputs in one
    lsg_gguf_mmvq_batch call: the six projections of one K run as one launch although they read
    three different activation rows; bits of the separate calls."""
    from layerstormgemmkernels_b200 import capi
    import ctypes
    t = T[name]
    K, KD = 1024, 3584
    # ("x" comes back after "att": the launch's matrices name their inputs one by one)
    shapes = [("x", 1024, K), ("x", 256, K), ("att", 1024, K), ("x", 256, K), ("h", 3584, K), ("h", 3584, K), ("act", 1024, KD)]
    g = torch.Generator().manual_seed(31 + M)
    xin = {}
    for grp, _, k in shapes:
        if grp not in xin:
            xin[grp] = (torch.randn(M, k, generator=g) * 0.5).to(torch.bfloat16).cuda()
    Ws = [torch.from_numpy(Q.random_gguf_weight(name, N, k, seed=7 + i)).cuda() for i, (_, N, k) in enumerate(shapes)]
    outs = [torch.zeros((M, N), dtype=torch.bfloat16, device="cuda") for _, N, _ in shapes]
    P = capi.GgufMmvqParams
    arr = (P * len(shapes))()
    for i, (grp, N, k) in enumerate(shapes):
        arr[i] = P(M=M, N=N, K=k, A=xin[grp].data_ptr(), B=Ws[i].data_ptr(), C=outs[i].data_ptr(), type=t,
                   out_dtype=capi.DTYPE_BF16)
    need = max(256, capi.lib.lsg_gguf_mmvq_batch_workspace_bytes(arr, len(shapes)))
    ws = torch.empty((need,), dtype=torch.uint8, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for _ in range(3):
        capi.check(capi.lib.lsg_gguf_mmvq_batch(arr, len(shapes), ctypes.c_void_p(ws.data_ptr()), need, st))
    torch.cuda.synchronize()
    for i, (grp, N, k) in enumerate(shapes):
        assert torch.equal(outs[i], ops.gguf_mmvq(xin[grp], Ws[i], t, N, k)), (i, grp)
    assert capi.device_status() == 0


def test_mmvq_batch_independent_launches_overlap_dependent_ones_wait(ops):
    """lsg_gguf_mmvq_batch lets a launch start before the one in front of it has finished when it
    shares no buffer with the earlier entries; an entry that reads an earlier result (or writes
    an earlier entry's buffer) must still wait.  Six entries in five launches of every kind (the
    plan is checked first), large enough to take a few microseconds each, replayed back to back
    from a CUDA graph with changing inputs: every result equals the separate calls'."""
    from layerstormgemmkernels_b200 import capi
    import ctypes
    t = T["Q4_K"]
    K0, N0, N1, N2 = 4096, 4096, 2048, 1024
    W0 = torch.from_numpy(Q.random_gguf_weight("Q4_K", N0, K0, seed=1)).cuda()     # 0: y0 = x W0^T
    W2 = torch.from_numpy(Q.random_gguf_weight("Q4_K", N2, K0, seed=3)).cuda()     # 1: y2 = x2 W2^T  (joins 0)
    W1 = torch.from_numpy(Q.random_gguf_weight("Q4_K", N1, N0, seed=2)).cuda()     # 2: y1 = y0 W1^T  (reads y0)
    W5 = torch.from_numpy(Q.random_gguf_weight("Q4_K", N2, N1, seed=6)).cuda()     # 3: y3 = x3 W5^T  (independent)
    W3 = torch.from_numpy(Q.random_gguf_weight("Q4_K", N2, N1, seed=4)).cuda()     # 4: y4 = y1 W3^T  (reads y1)
    W4 = torch.from_numpy(Q.random_gguf_weight("Q4_K", N2, K0, seed=5)).cuda()     # 5: y2 = x W4^T   (rewrites y2)
    x = torch.zeros((1, K0), dtype=torch.bfloat16, device="cuda")
    x2 = torch.zeros((1, K0), dtype=torch.bfloat16, device="cuda")
    x3 = torch.zeros((1, N1), dtype=torch.bfloat16, device="cuda")
    y0 = torch.zeros((1, N0), dtype=torch.bfloat16, device="cuda")
    y1 = torch.zeros((1, N1), dtype=torch.bfloat16, device="cuda")
    y2 = torch.zeros((1, N2), dtype=torch.bfloat16, device="cuda")
    y3 = torch.zeros((1, N2), dtype=torch.bfloat16, device="cuda")
    y4 = torch.zeros((1, N2), dtype=torch.bfloat16, device="cuda")
    P = capi.GgufMmvqParams
    arr = (P * 6)()
    mk = lambda N, K, A, W, C: P(M=1, N=N, K=K, A=A.data_ptr(), B=W.data_ptr(), C=C.data_ptr(), type=t,  # noqa: E731
                                 out_dtype=capi.DTYPE_BF16)
    arr[0] = mk(N0, K0, x, W0, y0)
    arr[1] = mk(N2, K0, x2, W2, y2)
    arr[2] = mk(N1, N0, y0, W1, y1)
    arr[3] = mk(N2, N1, x3, W5, y3)
    arr[4] = mk(N2, N1, y1, W3, y4)
    arr[5] = mk(N2, K0, x, W4, y2)
    f, c, k = (ctypes.c_int * 8)(), (ctypes.c_int * 8)(), (ctypes.c_int * 8)()
    n = capi.lib.lsg_gguf_mmvq_batch_plan(arr, 6, f, c, k, 8)
    assert [(f[i], c[i], k[i]) for i in range(n)] == [(0, 2, 1), (2, 1, 0), (3, 1, 2), (4, 1, 0), (5, 1, 0)]
    need = max(256, capi.lib.lsg_gguf_mmvq_batch_workspace_bytes(arr, 6))
    ws = torch.empty((need,), dtype=torch.uint8, device="cuda")

    def batch():
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        capi.check(capi.lib.lsg_gguf_mmvq_batch(arr, 6, ctypes.c_void_p(ws.data_ptr()), need, st))

    g = torch.Generator().manual_seed(9)
    xs = [(torch.randn(1, K0, generator=g) * 0.5).to(torch.bfloat16).cuda() for _ in range(6)]
    batch()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph):
            batch()
    for it in range(6):
        x.copy_(xs[it])
        x2.copy_(xs[(it + 1) % 6])
        x3.copy_(xs[(it + 2) % 6][:, :N1])
        for _ in range(3):      # back-to-back replays: the next batch's first launch follows the last one directly
            graph.replay()
        torch.cuda.synchronize()
        r0 = ops.gguf_mmvq(xs[it], W0, t, N0, K0)
        r1 = ops.gguf_mmvq(r0, W1, t, N1, N0)
        assert torch.equal(y0, r0) and torch.equal(y1, r1)
        assert torch.equal(y3, ops.gguf_mmvq(x3, W5, t, N2, N1))
        assert torch.equal(y4, ops.gguf_mmvq(r1, W3, t, N2, N1))
        assert torch.equal(y2, ops.gguf_mmvq(xs[it], W4, t, N2, K0))
    assert capi.device_status() == 0


@pytest.mark.parametrize("name,M,K,Ns", [
    ("Q4_K", 1, 4096, (4096, 1024, 1024)),       # q, k, v
    ("Q4_K", 1, 4096, (14336, 14336)),           # gate, up
    ("Q6_K", 3, 1024, (96, 7, 640, 33)),         # four matrices, ragged and tiny ones
    ("Q8_0", 9, 512, (1, 300)),                  # more rows than one register pass
    ("Q4_K", 40, 1024, (200, 120)),              # more rows than one launch holds
    ("Q4_0", 2, 2048, (513, 511, 2, 2, 700)),    # five entries: a launch of four, then one
])
def test_mmvq_batch_joined_launch_equals_separate_calls(ops, name, M, K, Ns):
    """lsg_gguf_mmvq_batch runs projections of one input as one launch; which CTA computes a
    row does not change its bits."""
    A = (torch.randn(M, K, generator=torch.Generator().manual_seed(17)) * 0.4).to(torch.bfloat16).cuda()
    Ws = [torch.from_numpy(Q.random_gguf_weight(name, N, K, seed=40 + i)).cuda() for i, N in enumerate(Ns)]
    for dt in (torch.bfloat16, torch.float32):
        outs = ops.gguf_mmvq_batch(A, [(W, N) for W, N in zip(Ws, Ns)], T[name], out_dtype=dt)
        for W, N, out in zip(Ws, Ns, outs):
            assert torch.equal(out, ops.gguf_mmvq(A, W, T[name], N, K, out_dtype=dt))


def test_mmvq_batch_matches_oracle(ops):
    name, M, K, Ns = "Q4_K", 2, 1024, (160, 96, 40)
    rng = np.random.default_rng(3)
    A = (torch.randn(M, K, generator=torch.Generator().manual_seed(19)) * 0.4).to(torch.bfloat16)
    Wn = [Q.random_gguf_weight(name, N, K, seed=50 + i) for i, N in enumerate(Ns)]
    outs = ops.gguf_mmvq_batch(A.cuda(), [(torch.from_numpy(W).cuda(), N) for W, N in zip(Wn, Ns)],
                               T[name], out_dtype=torch.float32)
    xq = oracle.quantize_q8_1(bf16_bits(A))
    for W, out in zip(Wn, outs):
        assert rel_err(out.cpu().numpy(), oracle.mmvq(T[name], xq, W, K)) <= TOL_F32


def test_mmvq_graph_capture(ops):
    """tests/test_gguf_mmvq.py:106-134: capture + replay equals eager."""
    N, K = 512, 1024
    A = (torch.randn(1, K, generator=torch.Generator().manual_seed(3)) * 0.4).to(torch.bfloat16).cuda()
    W = torch.from_numpy(Q.random_gguf_weight("Q8_0", N, K, seed=11)).cuda()
    eager = ops.gguf_mmvq(A, W, T["Q8_0"], N, K)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            ops.gguf_mmvq(A, W, T["Q8_0"], N, K)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        captured = ops.gguf_mmvq(A, W, T["Q8_0"], N, K)
    captured.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(eager, captured)


def test_mmvq_full_size_linearity(ops):
    """Llama-3-8B gate/up shape (14336 x 4096, Q4_K): too big for the scalar oracle, so
    check size-independent properties: a sampled set of rows against the oracle, and
    exact agreement between M=1 calls and the rows of an M=8 call."""
    N, K = 14336, 4096
    W = Q.random_gguf_weight("Q4_K", N, K, seed=5)
    Wd = torch.from_numpy(W).cuda()
    A = torch.randn(8, K, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).cuda()
    y8 = ops.gguf_mmvq(A, Wd, T["Q4_K"], N, K, out_dtype=torch.float32).cpu().numpy()
    rows = np.r_[0:8, 7000:7008, N - 8:N]
    ref = oracle.mmvq(T["Q4_K"], oracle.quantize_q8_1(bf16_bits(A)), W[rows], K)
    assert rel_err(y8[:, rows], ref) <= TOL_F32
    y1 = ops.gguf_mmvq(A[3:4].contiguous(), Wd, T["Q4_K"], N, K, out_dtype=torch.float32).cpu().numpy()
    assert rel_err(y1[0], y8[3].astype(np.float64)) <= TOL_F32


def test_errors_mirror_reference(ops):
    A = torch.zeros(1, 100, dtype=torch.bfloat16, device="cuda")
    W = torch.zeros(8, 144, dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError, match="divisible"):      # std::invalid_argument -> ValueError
        ops.gguf_mmvq(A, W, T["Q4_K"], 8, 100)
    with pytest.raises(RuntimeError, match="BF16"):         # TORCH_CHECK -> RuntimeError
        ops.gguf_mmvq(A.float(), W, T["Q4_K"], 8, 100)
    with pytest.raises(RuntimeError, match="size"):
        ops.gguf_mmvq(A, W, T["Q4_K"], 8, 256)


@pytest.mark.parametrize("warps,ctas,stage_kib,share", [
    (15, 1, 1, 1),     # many warps, tiny stages: claims run laps ahead of the ring
    (11, 1, 16, 2), (3, 4, 4, 4), (1, 1, 2, 1), (7, 2, 8, 2), (15, 1, 64, 1),
])
def test_mmvq_results_do_not_depend_on_launch_geometry(ops, warps, ctas, stage_kib, share):
    """The pipeline (ring depth, work queue, CTA count) must never change a result."""
    from layerstormgemmkernels_b200 import capi
    cases = [("Q4_K", 2000, 4096, 1), ("Q4_K", 500, 14336, 1), ("Q6_K", 1111, 4096, 3),
             ("Q8_0", 300, 1024, 8), ("Q4_K", 700, 768, 2)]
    try:
        for name, N, K, M in cases:
            t = T[name]
            A = torch.randn(M, K, generator=torch.Generator().manual_seed(N)).to(torch.bfloat16).cuda()
            W = Q.random_gguf_weight(name, N, K, seed=K + N)
            Wd = torch.from_numpy(W).cuda()
            capi.check(capi.lib.lsg_mmvq_set_tuning(15, 1, 24, 1, 0))
            base = ops.gguf_mmvq(A, Wd, t, N, K, out_dtype=torch.float32)
            capi.check(capi.lib.lsg_mmvq_set_tuning(warps, ctas, stage_kib, share, 0))
            for _ in range(3):
                got = ops.gguf_mmvq(A, Wd, t, N, K, out_dtype=torch.float32)
                assert torch.equal(base, got), (name, N, K, M)
            if name == "Q4_K" and N == 2000:
                ref = oracle.mmvq(t, oracle.quantize_q8_1(bf16_bits(A)), W, K)
                assert rel_err(got.cpu().numpy(), ref) <= TOL_F32
        assert capi.device_status() == 0
    finally:
        capi.check(capi.lib.lsg_mmvq_set_tuning(15, 1, 24, 1, 0))
