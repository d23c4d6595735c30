"""GPU tests of the grouped (MoE) GEMM and its device-side routing metadata.  The cases
restate tests/test_gguf_grouped_gemm.py of the reference; the checker is the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle
from layerstormgemmkernels_b200 import quantize as Q
from layerstormgemmkernels_b200.capi import GGUF_TYPES

pytestmark = pytest.mark.gpu
T = GGUF_TYPES
REF_TYPES = ["Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "Q8_0", "MXFP4"]
F_AUTO, F_MMVQ, F_MMQ, F_HOSTLOOP = 0, 1, 2, 3
S_DEQUANT, S_INT = 0, 1
TOL_F32 = 2e-5


@pytest.fixture(scope="module")
def ops():
    from layerstormgemmkernels_b200 import ops as _ops, capi
    yield _ops
    assert capi.device_status() == 0


def bits_of(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def build_group(name, counts, N, K, seed=0):
    E = len(counts)
    offs = np.zeros(E + 1, dtype=np.int32)
    offs[1:] = np.cumsum(counts)
    A = (torch.randn(int(offs[-1]), K, generator=torch.Generator().manual_seed(seed)) * 0.4
         ).to(torch.bfloat16).cuda()
    host_w = [Q.random_gguf_weight(name, N, K, seed + 1 + e) for e in range(E)]
    dev_w = [torch.from_numpy(w).cuda() for w in host_w]
    ptrs = torch.tensor([w.data_ptr() for w in dev_w], dtype=torch.int64, device="cuda")
    return A, torch.from_numpy(offs).cuda(), ptrs, dev_w, host_w, offs


def oracle_grouped(name, A, host_w, offs, K, dequant=False):
    t = T[name]
    N = host_w[0].shape[0]
    out = np.full((int(offs[-1]), N), np.nan)
    b = bits_of(A)
    for e, W in enumerate(host_w):
        s, en = int(offs[e]), int(offs[e + 1])
        if s == en:
            continue
        if dequant:
            out[s:en] = oracle.dequant_gemm(t, b[s:en], W, K)
        else:
            out[s:en] = oracle.mmvq(t, oracle.quantize_q8_1(b[s:en]), W, K)
    return out


def check(got, ref, tol):
    live = ~np.isnan(ref)
    scale = np.abs(ref[live]).max()
    assert np.abs(got[live] - ref[live]).max() <= tol * scale


DISTS = {
    "decode": lambda E: [1 + (e % 8) for e in range(E)],
    "prefill": lambda E: [64 + 40 * (e % 4) for e in range(E)],
    "mixed": lambda E: [(2 if e % 2 == 0 else 96 + 20 * (e % 3)) for e in range(E)],
    "empty": lambda E: [0 if e % 3 == 0 else (1 + (e % 7)) for e in range(E)],
}


@pytest.mark.parametrize("name", REF_TYPES + ["Q4_0"])
@pytest.mark.parametrize("dist", list(DISTS))
def test_grouped_int_vs_oracle(ops, name, dist):
    """tests/test_gguf_grouped_gemm.py:129-159, with the oracle as the golden."""
    E, K, N = 6, 256, 256
    A, off, ptrs, dev_w, host_w, offs = build_group(name, DISTS[dist](E), N, K, seed=100)
    ref = oracle_grouped(name, A, host_w, offs, K)
    outs = {}
    tensor_cores_by_default = int(offs[-1]) // E > 8     # the reference's auto rule
    for label, force in (("auto", F_AUTO), ("mmvq", F_MMVQ), ("mmq", F_MMQ), ("hostloop", F_HOSTLOOP)):
        outs[label] = ops.gguf_grouped_gemm(A, off, ptrs, T[name], S_INT, N, K, force,
                                            out_dtype=torch.float32).cpu().numpy()
        # mat-vec kernels: summation order only (2e-5); tensor-core path: fp16 operands, held
        # to the north-star GEMM bound of 1e-3 of the output scale
        on_tc = label == "mmq" or (label == "auto" and tensor_cores_by_default)
        check(outs[label], ref, 1e-3 if on_tc else TOL_F32)
    # lossless-activation golden through the host loop
    gold = ops.gguf_grouped_gemm(A, off, ptrs, T[name], S_DEQUANT, N, K, F_HOSTLOOP,
                                 out_dtype=torch.float32).cpu().numpy()
    check(gold, oracle_grouped(name, A, host_w, offs, K, dequant=True), TOL_F32)
    live = ~np.isnan(ref)
    a, b = gold[live], outs["auto"][live]
    assert (a * b).sum() / np.sqrt((a * a).sum() * (b * b).sum()) >= 0.999
    # bf16 output = rounding of the fp32 accumulator
    o16 = ops.gguf_grouped_gemm(A, off, ptrs, T[name], S_INT, N, K, F_AUTO)
    exp = torch.from_numpy(outs["auto"]).to(torch.bfloat16)
    lv = torch.from_numpy(live)
    assert torch.equal(o16.cpu()[lv], exp[lv])


@pytest.mark.parametrize("name", REF_TYPES)
@pytest.mark.parametrize("m", [1, 3, 8, 12])
def test_grouped_single_expert_and_determinism(ops, name, m):
    """tests/test_gguf_grouped_gemm.py:173-195."""
    K, N = 512, 384
    A, off, ptrs, dev_w, host_w, offs = build_group(name, [m], N, K, seed=300)
    ref = oracle_grouped(name, A, host_w, offs, K)
    out = ops.gguf_grouped_gemm(A, off, ptrs, T[name], S_INT, N, K, F_MMVQ, out_dtype=torch.float32)
    check(out.cpu().numpy(), ref, TOL_F32)
    out2 = ops.gguf_grouped_gemm(A, off, ptrs, T[name], S_INT, N, K, F_MMVQ, out_dtype=torch.float32)
    assert torch.equal(out, out2)
    # the single-weight operator computes the same thing
    single = ops.gguf_mmvq(A, dev_w[0], T[name], N, K, out_dtype=torch.float32)
    check(single.cpu().numpy(), ref, TOL_F32)


@pytest.mark.parametrize("name", ["Q8_0", "Q4_K", "Q6_K"])
def test_grouped_topk_like_counts(ops, name):
    """Uneven counts as top-k routing produces (tests/test_gguf_grouped_gemm.py:202-221)."""
    E, K, N = 16, 512, 320
    rng = np.random.default_rng(5)
    counts = np.bincount(rng.integers(0, E, size=40), minlength=E).tolist()
    A, off, ptrs, dev_w, host_w, offs = build_group(name, counts, N, K, seed=500)
    ref = oracle_grouped(name, A, host_w, offs, K)
    out = ops.gguf_grouped_gemm(A, off, ptrs, T[name], S_INT, N, K, F_AUTO, out_dtype=torch.float32)
    check(out.cpu().numpy(), ref, TOL_F32)


def test_grouped_moe_config_shapes(ops):
    """The MoE config's projections (128 experts, H=2048, I=768, Q4_K) at T=1 and T=64
    tokens x top-8: sampled experts against the oracle."""
    E = 128
    for (N, K) in ((768, 2048), (2048, 768)):
        for tokens in (1, 64):
            rng = np.random.default_rng(tokens + N)
            idx = np.concatenate([rng.choice(E, 8, replace=False) for _ in range(tokens)])
            counts = np.bincount(idx, minlength=E).tolist()
            base = Q.random_gguf_weight("Q4_K", N, K, 7)
            host_w = []
            for e in range(E):
                w = base.copy()
                w[:, 16:24] = (e * 37 + np.arange(8)) % 251      # make experts differ cheaply
                host_w.append(w)
            dev_w = [torch.from_numpy(w).cuda() for w in host_w]
            ptrs = torch.tensor([w.data_ptr() for w in dev_w], dtype=torch.int64, device="cuda")
            offs = np.zeros(E + 1, dtype=np.int32)
            offs[1:] = np.cumsum(counts)
            A = torch.randn(int(offs[-1]), K, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).cuda()
            out = ops.gguf_grouped_gemm(A, torch.from_numpy(offs).cuda(), ptrs, T["Q4_K"], S_INT, N, K,
                                        F_AUTO, out_dtype=torch.float32).cpu().numpy()
            b = bits_of(A)
            live = [e for e in range(E) if counts[e] > 0]
            for e in live[:3] + live[-3:]:
                s, en = int(offs[e]), int(offs[e + 1])
                ref = oracle.mmvq(T["Q4_K"], oracle.quantize_q8_1(b[s:en]), host_w[e], K)
                assert np.abs(out[s:en] - ref).max() <= TOL_F32 * np.abs(ref).max()


def test_null_expert_pointer_is_skipped(ops):
    A, off, ptrs, dev_w, host_w, offs = build_group("Q4_K", [2, 3, 4], 128, 256, seed=9)
    ptrs2 = ptrs.clone()
    ptrs2[1] = 0
    D = ops.gguf_grouped_gemm(A, off, ptrs2, T["Q4_K"], S_INT, 128, 256, F_AUTO, out_dtype=torch.float32)
    ref = oracle_grouped("Q4_K", A, host_w, offs, 256)
    got = D.cpu().numpy()
    for e in (0, 2):
        s, en = int(offs[e]), int(offs[e + 1])
        assert np.abs(got[s:en] - ref[s:en]).max() <= TOL_F32 * np.abs(ref[s:en]).max()


def test_grouped_graph_capture(ops):
    """tests/test_gguf_grouped_gemm.py:227-261: the device-routed path captures and replays."""
    A, off, ptrs, dev_w, host_w, offs = build_group("Q4_K", [3, 0, 5, 1], 256, 512, seed=11)
    eager = ops.gguf_grouped_gemm(A, off, ptrs, T["Q4_K"], S_INT, 256, 512, F_AUTO)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            ops.gguf_grouped_gemm(A, off, ptrs, T["Q4_K"], S_INT, 256, 512, F_AUTO)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        captured = ops.gguf_grouped_gemm(A, off, ptrs, T["Q4_K"], S_INT, 256, 512, F_AUTO)
    captured.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(eager, captured)


@pytest.mark.parametrize("counts", [[0, 0, 0], [5], [1, 0, 3, 0, 0, 200, 64, 65], list(range(70)),
                                    [0] * 40 + [7] + [0] * 30 + [129]])
def test_routing_metadata_bit_exact(ops, counts):
    """Active-expert list and m-tile map against their definitions
    (gguf_grouped_int.cu:46-66, 156-187)."""
    E = len(counts)
    offs = np.zeros(E + 1, dtype=np.int32)
    offs[1:] = np.cumsum(counts)
    Tt = int(offs[-1])
    off_d = torch.from_numpy(offs).cuda()
    for cap in {max(1, min(E, Tt)), E, 3}:
        act = [e for e in range(E) if counts[e] > 0][:cap]
        want = np.array(act + [-1] * (cap - len(act)), dtype=np.int32)
        np.testing.assert_array_equal(ops.build_active_expert_list(off_d, cap).cpu().numpy(), want)
    for tile_m in (64, 128):
        t_max = (Tt + tile_m - 1) // tile_m + E
        te, tm = [], []
        for e in range(E):
            for i in range((counts[e] + tile_m - 1) // tile_m):
                te.append(e)
                tm.append(int(offs[e]) + i * tile_m)
        te += [-1] * (t_max - len(te))
        tm += [0] * (t_max - len(tm))
        g_te, g_tm = ops.build_mmq_tile_map(off_d, tile_m, t_max)
        np.testing.assert_array_equal(g_te.cpu().numpy(), np.array(te, np.int32))
        np.testing.assert_array_equal(g_tm.cpu().numpy(), np.array(tm, np.int32))


def test_grouped_errors(ops):
    A = torch.zeros(4, 100, dtype=torch.bfloat16, device="cuda")
    off = torch.tensor([0, 4], dtype=torch.int32, device="cuda")
    ptrs = torch.tensor([A.data_ptr()], dtype=torch.int64, device="cuda")
    with pytest.raises(Exception, match="divisible"):
        ops.gguf_grouped_gemm(A, off, ptrs, T["Q4_K"], S_INT, 8, 100)
    with pytest.raises(RuntimeError, match="int32"):
        ops.gguf_grouped_gemm(A, off.long(), ptrs, T["Q4_K"], S_INT, 8, 100)
    # empty problem returns silently
    A0 = torch.zeros(0, 256, dtype=torch.bfloat16, device="cuda")
    off0 = torch.tensor([0, 0], dtype=torch.int32, device="cuda")
    assert ops.gguf_grouped_gemm(A0, off0, ptrs, T["Q4_K"], S_INT, 8, 256).shape == (0, 8)


# ---------------------------------------------------------------------------
# Tensor-core (tcgen05) path
# ---------------------------------------------------------------------------
TOL_TC = 1e-3   # the north-star GEMM bound: max |y - ref| / max |ref|


@pytest.mark.parametrize("name,M,N,K", [
    ("Q4_K", 128, 256, 256), ("Q4_K", 300, 512, 1024), ("Q6_K", 129, 320, 512),
    ("Q8_0", 64, 256, 96), ("Q4_0", 200, 1000, 4096), ("Q5_K", 257, 264, 768),
    ("Q2_K", 17, 256, 256), ("Q3_K", 500, 136, 512), ("MXFP4", 130, 256, 128),
])
def test_mmq_dense_vs_oracle(ops, name, M, N, K):
    t = T[name]
    A = (torch.randn(M, K, generator=torch.Generator().manual_seed(M + N)) * 0.4).to(torch.bfloat16).cuda()
    W = Q.random_gguf_weight(name, N, K, seed=K)
    Wd = torch.from_numpy(W).cuda()
    ref = oracle.mmvq(t, oracle.quantize_q8_1(bits_of(A)), W, K)
    got = ops.gguf_mmq(A, Wd, t, N, K, out_dtype=torch.float32).cpu().numpy()
    assert np.abs(got - ref).max() <= TOL_TC * np.abs(ref).max()
    # the mat-vec path computes the same numbers
    mv = ops.gguf_mmvq(A, Wd, t, N, K, out_dtype=torch.float32).cpu().numpy()
    assert np.abs(got - mv).max() <= TOL_TC * np.abs(ref).max()
    g16 = ops.gguf_mmq(A, Wd, t, N, K).float().cpu().numpy()
    assert np.abs(g16 - ref).max() <= (TOL_TC + 2.0 ** -8) * np.abs(ref).max()


def test_mmq_prefill_config_shape_sampled(ops):
    """Prefill config: Q4_K 14336 x 4096, M = 512; sampled rows/columns against the oracle."""
    N, K, M = 14336, 4096, 512
    A = torch.randn(M, K, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).cuda()
    W = Q.random_gguf_weight("Q4_K", N, K, seed=2)
    got = ops.gguf_mmq(A, torch.from_numpy(W).cuda(), T["Q4_K"], N, K, out_dtype=torch.float32).cpu().numpy()
    rows = np.r_[0:4, 250:254, 508:512]
    cols = np.r_[0:8, 7000:7008, N - 8:N]
    ref = oracle.mmvq(T["Q4_K"], oracle.quantize_q8_1(bits_of(A)[rows]), W[cols], K)
    assert np.abs(got[np.ix_(rows, cols)] - ref).max() <= TOL_TC * np.abs(ref).max()


def test_grouped_many_experts_takes_the_global_tile_lookup(ops):
    """More token tiles than the fused kernel's shared-memory tile table holds (340): 400 experts with
    9..40 rows each take 64-row tiles, one or more per expert, and every role then resolves its
    tiles from global memory.  Same results as the oracle; balanced tiles (33..40 rows stay one
    tile, nothing is split unevenly) and empty experts included."""
    E, K, N = 400, 256, 128
    counts = [0 if e % 50 == 7 else 9 + (e * 7) % 32 for e in range(E)]
    A, off, ptrs, dev_w, host_w, offs = build_group("Q4_K", counts, N, K, seed=900)
    ref = oracle_grouped("Q4_K", A, host_w, offs, K)
    out = ops.gguf_grouped_gemm(A, off, ptrs, T["Q4_K"], S_INT, N, K, F_MMQ, out_dtype=torch.float32)
    check(out.cpu().numpy(), ref, TOL_TC)


@pytest.mark.parametrize("rows", [257, 320, 321, 384, 385, 700])
def test_grouped_tall_and_balanced_tiles(ops, rows):
    """Experts around the tile heights of the fused kernel: one 320- or 384-row tile, two evenly
    shared tiles just above it, and several tiles for a large expert, next to a small and an empty one."""
    K, N = 512, 256
    counts = [rows, 0, 5, rows - 1]
    A, off, ptrs, dev_w, host_w, offs = build_group("Q4_K", counts, N, K, seed=rows)
    ref = oracle_grouped("Q4_K", A, host_w, offs, K)
    out = ops.gguf_grouped_gemm(A, off, ptrs, T["Q4_K"], S_INT, N, K, F_MMQ, out_dtype=torch.float32)
    check(out.cpu().numpy(), ref, TOL_TC)
    again = ops.gguf_grouped_gemm(A, off, ptrs, T["Q4_K"], S_INT, N, K, F_MMQ, out_dtype=torch.float32)
    assert torch.equal(out, again)
