"""GPU tests of the tensor-core GEMM that decodes the packed weights inside the kernel
(weight rows on the 128-lane side, tokens on the N side, optional split of K).  The
checker is the CPU oracle of the reference's integer path (gguf_mmvq.cu:66-187 after
quantize_bf16_to_q8_1); the bound is the GEMM tolerance max|y - ref| <= 1e-3 max|ref|."""
import numpy as np
import pytest
import torch

import oracle
from layerstormgemmkernels_b200 import quantize as Q
from layerstormgemmkernels_b200.capi import GGUF_TYPES

pytestmark = pytest.mark.gpu
T = GGUF_TYPES
ALL_TYPES = ["Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "Q8_0", "MXFP4", "Q4_0"]
TOL_TC = 1e-3


@pytest.fixture(scope="module")
def ops():
    from layerstormgemmkernels_b200 import ops as _ops, capi
    yield _ops
    capi.check(capi.lib.lsg_mmq_set_weight_path(-1))
    assert capi.device_status() == 0


@pytest.fixture
def weight_path():
    from layerstormgemmkernels_b200 import capi

    def set_mode(mode):
        capi.check(capi.lib.lsg_mmq_set_weight_path(mode))
    yield set_mode
    capi.check(capi.lib.lsg_mmq_set_weight_path(-1))


def bits_of(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def make_case(name, M, N, K, seed):
    A = (torch.randn(M, K, generator=torch.Generator().manual_seed(seed)) * 0.4).to(torch.bfloat16).cuda()
    W = Q.random_gguf_weight(name, N, K, seed=seed + 1)
    return A, W, torch.from_numpy(W).cuda()


@pytest.mark.parametrize("name", ALL_TYPES)
@pytest.mark.parametrize("M,N,K", [(1, 128, 256), (5, 200, 512), (33, 384, 256), (129, 130, 768), (300, 256, 1024)])
def test_fused_dense_every_type_vs_oracle(ops, weight_path, name, M, N, K):
    weight_path(2)
    A, W, Wd = make_case(name, M, N, K, seed=M + N)
    ref = oracle.mmvq(T[name], oracle.quantize_q8_1(bits_of(A)), W, K)
    got = ops.gguf_mmq(A, Wd, T[name], N, K, out_dtype=torch.float32).cpu().numpy()
    assert got.shape == (M, N)
    assert np.abs(got - ref).max() <= TOL_TC * np.abs(ref).max()
    g16 = ops.gguf_mmq(A, Wd, T[name], N, K).float().cpu().numpy()
    assert np.abs(g16 - ref).max() <= (TOL_TC + 2.0 ** -8) * np.abs(ref).max()


@pytest.mark.parametrize("name", ["Q8_0", "Q4_0", "MXFP4"])
def test_fused_k_not_a_multiple_of_64(ops, weight_path, name):
    """32-value block types allow K = 32 (mod 64): the last K block is half empty."""
    weight_path(2)
    M, N, K = 20, 256, 96
    A, W, Wd = make_case(name, M, N, K, seed=9)
    ref = oracle.mmvq(T[name], oracle.quantize_q8_1(bits_of(A)), W, K)
    got = ops.gguf_mmq(A, Wd, T[name], N, K, out_dtype=torch.float32).cpu().numpy()
    assert np.abs(got - ref).max() <= TOL_TC * np.abs(ref).max()


@pytest.mark.parametrize("M", [2, 4, 8, 16, 40])
@pytest.mark.parametrize("N,K", [(1024, 4096), (4096, 4096), (512, 14336)])
def test_fused_q4k_decode_batches_split_k(ops, weight_path, M, N, K):
    """Few tokens and few weight tiles: K is split over CTAs and the partial tiles are added
    in split order by the last arrival, so two runs agree bit for bit."""
    weight_path(1)
    A, W, Wd = make_case("Q4_K", M, N, K, seed=M)
    got = ops.gguf_mmq(A, Wd, T["Q4_K"], N, K, out_dtype=torch.float32)
    again = ops.gguf_mmq(A, Wd, T["Q4_K"], N, K, out_dtype=torch.float32)
    assert torch.equal(got, again)
    cols = np.r_[0:16, N // 2:N // 2 + 16, N - 16:N]
    ref = oracle.mmvq(T["Q4_K"], oracle.quantize_q8_1(bits_of(A)), W[cols], K)
    assert np.abs(got.cpu().numpy()[:, cols] - ref).max() <= TOL_TC * np.abs(ref).max()
    # the mat-vec kernel computes the same numbers from the same Q8_1 activations
    mv = ops.gguf_mmvq(A, Wd, T["Q4_K"], N, K, out_dtype=torch.float32)
    assert (got - mv).abs().max().item() <= TOL_TC * np.abs(ref).max()


def test_fused_and_prepared_weight_paths_agree(ops, weight_path):
    M, N, K = 260, 640, 2048
    A, W, Wd = make_case("Q4_K", M, N, K, seed=4)
    outs = []
    for mode in (0, 1, 2):
        weight_path(mode)
        outs.append(ops.gguf_mmq(A, Wd, T["Q4_K"], N, K, out_dtype=torch.float32))
    scale = outs[0].abs().max().item()
    assert (outs[0] - outs[1]).abs().max().item() <= TOL_TC * scale
    assert (outs[0] - outs[2]).abs().max().item() <= TOL_TC * scale


def test_fused_q4k_matrix_at_an_odd_address(ops, weight_path):
    """The staged Q4_K decoder copies 16-byte pieces and needs 16-byte alignment; a matrix
    that starts at another address goes through the byte-wise decoder (fp32 arithmetic,
    one rounding to fp16) and agrees to the fp16 rounding of the weights."""
    weight_path(1)
    M, N, K = 24, 256, 512
    A, W, Wd = make_case("Q4_K", M, N, K, seed=21)
    aligned = ops.gguf_mmq(A, Wd, T["Q4_K"], N, K, out_dtype=torch.float32)
    buf = torch.zeros(Wd.numel() + 64, dtype=torch.uint8, device="cuda")
    shifted = buf[6:6 + Wd.numel()]
    shifted.copy_(Wd.reshape(-1))
    assert shifted.data_ptr() % 16 != 0
    moved = ops.gguf_mmq(A, shifted.view(N, -1), T["Q4_K"], N, K, out_dtype=torch.float32)
    scale = aligned.abs().max().item()
    assert (aligned - moved).abs().max().item() <= TOL_TC * scale
    ref = oracle.mmvq(T["Q4_K"], oracle.quantize_q8_1(bits_of(A)), W, K)
    assert np.abs(moved.cpu().numpy() - ref).max() <= TOL_TC * np.abs(ref).max()


@pytest.mark.parametrize("name", ALL_TYPES)
def test_fused_grouped_every_type(ops, weight_path, name):
    """Expert-routed tiles through the fused kernel (reference: launch_gguf_grouped_gemm_int
    with force = mmq, gguf_grouped_int.cu:930-1010)."""
    weight_path(2)
    E, K, N = 5, 512, 320
    counts = [70, 0, 3, 130, 257]
    offs = np.zeros(E + 1, dtype=np.int32)
    offs[1:] = np.cumsum(counts)
    A = (torch.randn(int(offs[-1]), K, generator=torch.Generator().manual_seed(5)) * 0.4).to(torch.bfloat16).cuda()
    host_w = [Q.random_gguf_weight(name, N, K, 50 + e) for e in range(E)]
    dev_w = [torch.from_numpy(w).cuda() for w in host_w]
    ptrs = torch.tensor([w.data_ptr() for w in dev_w], dtype=torch.int64, device="cuda")
    out = ops.gguf_grouped_gemm(A, torch.from_numpy(offs).cuda(), ptrs, T[name], 1, N, K, 2,
                                out_dtype=torch.float32).cpu().numpy()
    xq = bits_of(A)
    for e in range(E):
        s, en = int(offs[e]), int(offs[e + 1])
        if s == en:
            continue
        ref = oracle.mmvq(T[name], oracle.quantize_q8_1(xq[s:en]), host_w[e], K)
        assert np.abs(out[s:en] - ref).max() <= TOL_TC * np.abs(ref).max()


def test_fused_prefill_config_shape_sampled(ops, weight_path):
    """Prefill config: Q4_K 14336 x 4096, M = 512; sampled rows/columns against the oracle."""
    weight_path(1)
    N, K, M = 14336, 4096, 512
    A = torch.randn(M, K, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).cuda()
    W = Q.random_gguf_weight("Q4_K", N, K, seed=2)
    got = ops.gguf_mmq(A, torch.from_numpy(W).cuda(), T["Q4_K"], N, K, out_dtype=torch.float32).cpu().numpy()
    rows = np.r_[0:4, 250:254, 508:512]
    cols = np.r_[0:8, 7000:7008, N - 8:N]
    ref = oracle.mmvq(T["Q4_K"], oracle.quantize_q8_1(bits_of(A)[rows]), W[cols], K)
    assert np.abs(got[np.ix_(rows, cols)] - ref).max() <= TOL_TC * np.abs(ref).max()


def _ffn_case(name, counts, H, I, seed):
    E = len(counts)
    offs = np.zeros(E + 1, dtype=np.int32)
    offs[1:] = np.cumsum(counts)
    A = (torch.randn(int(offs[-1]), H, generator=torch.Generator().manual_seed(seed)) * 0.5).to(torch.bfloat16).cuda()
    # real quantized weights of N(0, 0.05): with random block bytes the activations of the second
    # GEMM leave the fp16 range of the tensor-core operands
    quant = {"Q4_K": Q.quantize_q4_k, "Q6_K": Q.quantize_q6_k, "Q8_0": Q.quantize_q8_0, "Q4_0": Q.quantize_q4_0}[name]
    rng = np.random.default_rng(seed)
    ws = [[torch.from_numpy(quant((rng.standard_normal((n, k)) * 0.05).astype(np.float32))).cuda()
           for (n, k) in ((I, H), (I, H), (H, I))] for e in range(E)]
    ptr = lambda j: torch.tensor([w[j].data_ptr() for w in ws], dtype=torch.int64, device="cuda")
    return A, torch.from_numpy(offs).cuda(), ws, ptr(0), ptr(1), ptr(2)


@pytest.mark.parametrize("name,counts", [
    ("Q4_K", [70, 0, 3, 130, 257]),      # tensor-core route, ragged tiles, an empty expert
    ("Q4_K", [2, 1, 0, 3]),              # few rows per expert: composed from the grouped mat-vec
    ("Q6_K", [40, 25, 0, 64]),           # no in-kernel decoder: composed route on tensor cores
    ("Q8_0", [9, 30]),
])
def test_moe_ffn_equals_three_grouped_gemms(ops, name, counts):
    """One-call expert block against the three grouped GEMMs with SwiGLU in between."""
    H, I = 512, 256
    A, offs, ws, gp, up, dp = _ffn_case(name, counts, H, I, seed=7)
    t = T[name]
    got = ops.gguf_moe_ffn(A, offs, gp, up, dp, t, H, I, out_dtype=torch.float32)
    g = ops.gguf_grouped_gemm(A, offs, gp, t, 1, I, H, 0)
    u = ops.gguf_grouped_gemm(A, offs, up, t, 1, I, H, 0)
    act = (torch.nn.functional.silu(g.float()) * u.float()).to(torch.bfloat16)
    ref = ops.gguf_grouped_gemm(act, offs, dp, t, 1, H, I, 0, out_dtype=torch.float32)
    live = torch.zeros(A.size(0), dtype=torch.bool, device="cuda")
    o = offs.cpu().numpy()
    for e in range(len(counts)):
        live[o[e]:o[e + 1]] = True
    scale = ref[live].abs().max().item()
    # both sides round gate/up to bf16 before the activation; a last-bit difference there moves
    # the activation by one bf16 ulp, hence the bf16-sized slack on top of the GEMM bound
    assert (got[live] - ref[live]).abs().max().item() <= (TOL_TC + 2.0 ** -8) * scale


def test_moe_ffn_matvec_threshold(ops):
    """lsg_gguf_moe_ffn_set_matvec_rows: with the threshold at -1 a batch of a few rows per expert
    runs on the tensor cores (tolerance against the mat-vec composition), and the default route
    is back, bit for bit, once the old value is restored."""
    from layerstormgemmkernels_b200 import capi
    H, I = 512, 256
    A, offs, ws, gp, up, dp = _ffn_case("Q4_K", [2, 1, 0, 3, 5, 0, 1, 4], H, I, seed=13)
    t = T["Q4_K"]
    base = ops.gguf_moe_ffn(A, offs, gp, up, dp, t, H, I, out_dtype=torch.float32)
    old = capi.lib.lsg_gguf_moe_ffn_set_matvec_rows(-1)
    try:
        assert old == 8
        tc = ops.gguf_moe_ffn(A, offs, gp, up, dp, t, H, I, out_dtype=torch.float32)
    finally:
        assert capi.lib.lsg_gguf_moe_ffn_set_matvec_rows(old) == -1
    again = ops.gguf_moe_ffn(A, offs, gp, up, dp, t, H, I, out_dtype=torch.float32)
    assert torch.equal(base, again)
    assert not torch.equal(base, tc)   # another route really ran
    # the two routes quantize the activation of the down projection from values that differ in
    # the last bf16 bit here and there; an int8 step of a block is 1/127 of its largest value
    scale = base.abs().max().item()
    assert (tc - base).abs().max().item() <= (TOL_TC + 2.0 ** -6) * scale


def test_moe_ffn_vs_oracle_small(ops):
    """End to end against the CPU oracle: Q8_1 mat-vec oracle for each projection, activation
    in fp32 with bf16 rounding in between."""
    name, H, I = "Q4_K", 256, 256
    counts = [20, 33]
    A, offs, ws, gp, up, dp = _ffn_case(name, counts, H, I, seed=11)
    got = ops.gguf_moe_ffn(A, offs, gp, up, dp, T[name], H, I, out_dtype=torch.float32).cpu().numpy()
    o = offs.cpu().numpy()
    for e in range(len(counts)):
        rows = slice(int(o[e]), int(o[e + 1]))
        wg, wu, wd = (w.cpu().numpy() for w in ws[e])
        xq = oracle.quantize_q8_1(bits_of(A)[rows])
        g = torch.from_numpy(oracle.mmvq(T[name], xq, wg, H).astype(np.float32)).to(torch.bfloat16)
        u = torch.from_numpy(oracle.mmvq(T[name], xq, wu, H).astype(np.float32)).to(torch.bfloat16)
        act = (torch.nn.functional.silu(g.float()) * u.float()).to(torch.bfloat16)
        ref = oracle.mmvq(T[name], oracle.quantize_q8_1(act.view(torch.int16).numpy().view(np.uint16)), wd, I)
        assert np.abs(got[rows] - ref).max() <= (TOL_TC + 2.0 ** -7) * np.abs(ref).max()


# ---------------------------------------------------------------------------
# Unquantized activations: bf16 x fp16 on the tensor core (legacy q4k_* operators)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("name,M,N,K", [
    ("Q4_K", 1, 256, 256), ("Q4_K", 7, 384, 1024), ("Q4_K", 64, 4096, 4096), ("Q4_K", 300, 200, 512),
    ("Q6_K", 33, 256, 512), ("Q8_0", 20, 130, 96), ("Q2_K", 5, 128, 256),
])
def test_gemm_bf16_activations_vs_dequant_oracle(ops, name, M, N, K):
    """C = A_bf16 . dequant(W)^T, checker = the fp32 dequant-then-matmul oracle
    (the reference's CPU path, tests/test_reference.py:284-329)."""
    A, W, Wd = make_case(name, M, N, K, seed=3 * M + N)
    cols = np.r_[0:min(N, 24), max(0, N - 24):N]
    ref = oracle.dequant_gemm(T[name], bits_of(A), W[cols], K)
    got = ops.gguf_gemm_bf16(A, Wd, T[name], N, K, out_dtype=torch.float32).cpu().numpy()[:, cols]
    assert np.abs(got - ref).max() <= TOL_TC * np.abs(ref).max()
    again = ops.gguf_gemm_bf16(A, Wd, T[name], N, K, out_dtype=torch.float32).cpu().numpy()[:, cols]
    assert np.array_equal(got, again)


def test_q4k_legacy_operators(ops):
    """q4k_dequant_gemm / q4k_cutlass_gemm of the reference (tests/test_kernels.py:736-820):
    same signature, bf16 output, argument checks."""
    M, N, K = 48, 512, 1024
    A = (torch.randn(M, K, generator=torch.Generator().manual_seed(1)) * 0.5).to(torch.bfloat16).cuda()
    W = Q.quantize_q4_k((np.random.default_rng(0).standard_normal((N, K)) * 0.02).astype(np.float32))
    Wd = torch.from_numpy(W).cuda()
    ref = oracle.dequant_gemm(T["Q4_K"], bits_of(A), W, K)
    for fn in (ops.q4k_dequant_gemm, ops.q4k_cutlass_gemm):
        out = fn(A, Wd)
        assert out.dtype == torch.bfloat16 and tuple(out.shape) == (M, N)
        assert np.abs(out.float().cpu().numpy() - ref).max() <= (TOL_TC + 2.0 ** -8) * np.abs(ref).max()
    with pytest.raises(RuntimeError):
        ops.q4k_dequant_gemm(A[:, :1000].contiguous(), Wd)          # K not a multiple of 256
    with pytest.raises(RuntimeError):
        ops.q4k_cutlass_gemm(A, Wd[:, :100].contiguous())            # row bytes mismatch


@pytest.mark.parametrize("M", [5, 300, 2100])      # split-K, fused, and prepared-operand routes
def test_mmq_gather_stores_every_tile_into_every_output(ops, M):
    """GEMM fused with the all-gather of a column-split weight: the slab's columns land at
    their offset in each output matrix (peers emulated by local buffers), nothing else is
    touched, and the values are those of gguf_mmq."""
    N_total, n_local, K, col0 = 640, 256, 512, 128
    A, W, Wd = make_case("Q4_K", M, n_local, K, seed=M)
    mmq = ops.gguf_mmq(A, Wd, T["Q4_K"], n_local, K)
    # the same route with a single plain output is the reference for the bits; above 2048 rows the
    # gather entry keeps the prepared-operand kernel while gguf_mmq decodes inside the GEMM, and
    # the two differ by the fp16 rounding of the weights
    ref = torch.empty((M, n_local), dtype=torch.bfloat16, device="cuda")
    ops.gguf_mmq_gather(A, Wd, T["Q4_K"], n_local, K, torch.tensor([ref.data_ptr()], dtype=torch.int64, device="cuda"),
                        n_local, 0)
    torch.cuda.synchronize()
    scale = mmq.float().abs().max().item()
    assert (ref.float() - mmq.float()).abs().max().item() <= (1e-3 + 2.0 ** -8) * scale
    if M <= 2048:
        assert torch.equal(ref, mmq)
    outs = [torch.full((M, N_total), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    ptrs = torch.tensor([o.data_ptr() for o in outs], dtype=torch.int64, device="cuda")
    ops.gguf_mmq_gather(A, Wd, T["Q4_K"], n_local, K, ptrs, N_total, col0)
    torch.cuda.synchronize()
    for o in outs:
        assert torch.equal(o[:, col0:col0 + n_local], ref)
        assert bool((o[:, :col0] == 7.0).all()) and bool((o[:, col0 + n_local:] == 7.0).all())
