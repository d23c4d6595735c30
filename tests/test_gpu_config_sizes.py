"""GPU parity at the full sizes of the benchmark configurations, checked on SAMPLED outputs
against the CPU oracle (the oracle needs seconds for a few thousand outputs, hours for all).

* prefill: Q4_K and Q6_K 14336 x 4096 at M = 512 and M = 4096 (the two kernels that serve
  them: weights decoded inside the GEMM up to 2048 rows, prepared operands above), sampled
  token rows x sampled weight rows against oracle.mmvq, bound 1e-3 of the largest |reference|.
* MoE layer: 128 experts, top-8, hidden 2048, expert FFN 768, Q4_K, T in {1, 64, 4096}: the
  whole layer (route -> permute -> gate|up -> SwiGLU -> down -> combine) on sampled tokens
  against oracle routing (the torch definition) + oracle.mmvq per expert + SwiGLU, bound 1e-3
  relative to the largest |reference| (plus one bf16 rounding of the output).
* NVFP4: 8 experts, top-2, hidden 4096, FFN 14336, 4096 tokens: gate projection and down
  projection on sampled rows x sampled columns against float64 dequantize-then-matmul
  (ref_nvfp4_dequant's definition, tests/test_reference.py:107-134 of the reference), bound 2e-2.

The reference's own cases at these shapes: tests/test_kernels.py:273-317, 543-652,
tests/test_gguf_grouped_gemm.py:129-159, 202-221 (small shapes there; the sizes here are the
benchmark's).
"""
import numpy as np
import pytest
import torch

import oracle
from layerstormgemmkernels_b200 import quantize as Q
from layerstormgemmkernels_b200.capi import GGUF_TYPES

pytestmark = pytest.mark.gpu
T = GGUF_TYPES


@pytest.fixture(scope="module")
def ops():
    from layerstormgemmkernels_b200 import ops as _ops, capi
    yield _ops
    assert capi.device_status() == 0


def bits_of(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def quantize_rows(name, w, threads=16):
    from concurrent.futures import ThreadPoolExecutor
    fn = Q.QUANTIZERS[name]
    chunks = np.array_split(np.arange(w.shape[0]), threads * 2)
    with ThreadPoolExecutor(max_workers=threads) as ex:
        return np.concatenate(list(ex.map(lambda idx: fn(w[idx[0]:idx[-1] + 1]), chunks)), axis=0)


@pytest.fixture(scope="module")
def prefill_weights():
    w = (torch.randn(14336, 4096, generator=torch.Generator().manual_seed(2)) * 0.02).numpy()
    return {name: quantize_rows(name, w) for name in ("Q4_K", "Q6_K")}


@pytest.mark.parametrize("name", ["Q4_K", "Q6_K"])
@pytest.mark.parametrize("M", [512, 4096])
def test_prefill_14336x4096_sampled_vs_oracle(ops, prefill_weights, name, M):
    N, K = 14336, 4096
    W = prefill_weights[name]
    A = torch.randn(M, K, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).cuda()
    got = ops.gguf_mmq(A, torch.from_numpy(W).cuda(), T[name], N, K, out_dtype=torch.float32).cpu().numpy()
    rng = np.random.default_rng(M)
    rows = np.unique(np.concatenate([[0, M - 1, 127, 128, 255, 256], rng.integers(0, M, 26)]))
    cols = np.unique(np.concatenate([[0, N - 1, 127, 128, 7167, 7168], rng.integers(0, N, 90)]))
    xq = oracle.quantize_q8_1(bits_of(A)[rows])
    ref = oracle.mmvq(T[name], xq, W[cols], K)
    err = np.abs(got[np.ix_(rows, cols)] - ref).max() / np.abs(ref).max()
    assert err <= 1e-3, (name, M, err)
    # bf16 output (what the reference operator returns)
    g16 = ops.gguf_mmq(A, torch.from_numpy(W).cuda(), T[name], N, K).float().cpu().numpy()
    err16 = np.abs(g16[np.ix_(rows, cols)] - ref).max() / np.abs(ref).max()
    assert err16 <= 1e-3 + 2.0 ** -8, (name, M, err16)


# ------------------------------------------------------------------------------------------
# MoE layer
# ------------------------------------------------------------------------------------------
E_MOE, K_MOE, H_MOE, I_MOE = 128, 8, 2048, 768


@pytest.fixture(scope="module")
def moe_weights():
    g = torch.Generator().manual_seed(3)
    base = []
    for _ in range(8):       # eight distinct experts, tiled over the 128 ids (as the benchmark)
        base.append((Q.quantize_q4_k((torch.randn(I_MOE, H_MOE, generator=g) * 0.02).numpy()),
                     Q.quantize_q4_k((torch.randn(I_MOE, H_MOE, generator=g) * 0.02).numpy()),
                     Q.quantize_q4_k((torch.randn(H_MOE, I_MOE, generator=g) * 0.02).numpy())))
    dev = [[torch.from_numpy(base[e % 8][j]).cuda() for e in range(E_MOE)] for j in range(3)]
    ptrs = [torch.tensor([w.data_ptr() for w in ws], dtype=torch.int64, device="cuda") for ws in dev]
    return base, dev, ptrs


def bf16_round(x):
    return torch.from_numpy(np.asarray(x, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def oracle_expert(base, e, x_bits_row):
    """One token through expert e as the reference's three Int-strategy grouped GEMMs with the
    activation computed in fp32 and stored as bf16 in between."""
    gw, uw, dw = base[e % 8]
    xq = oracle.quantize_q8_1(x_bits_row[None, :])
    g = bf16_round(oracle.mmvq(T["Q4_K"], xq, gw, H_MOE)[0])
    u = bf16_round(oracle.mmvq(T["Q4_K"], xq, uw, H_MOE)[0])
    act = bf16_round((g / (1.0 + np.exp(-g.astype(np.float32)))) * u)
    act_bits = torch.from_numpy(act).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    aq = oracle.quantize_q8_1(act_bits[None, :])
    return bf16_round(oracle.mmvq(T["Q4_K"], aq, dw, I_MOE)[0])


@pytest.mark.parametrize("tokens", [1, 64, 4096])
def test_moe_layer_128_experts_top8_sampled_vs_oracle(ops, moe_weights, tokens):
    base, _dev, (gate_p, up_p, down_p) = moe_weights
    g = torch.Generator().manual_seed(100 + tokens)
    hidden = torch.randn(tokens, H_MOE, generator=g).to(torch.bfloat16)
    logits = torch.randn(tokens, E_MOE, generator=g)
    h_dev, l_dev = hidden.cuda(), logits.cuda()
    idx, w = ops.moe_route(l_dev, K_MOE)
    offs, perm, inv = ops.moe_permutation(idx, E_MOE)
    rows = ops.moe_permute(h_dev, perm, K_MOE)
    y = ops.gguf_moe_ffn(rows, offs, gate_p, up_p, down_p, T["Q4_K"], H_MOE, I_MOE)
    # the same block with the gather folded in must give the same bits
    y_fused = ops.gguf_moe_ffn(h_dev, offs, gate_p, up_p, down_p, T["Q4_K"], H_MOE, I_MOE, perm=perm, top_k=K_MOE)
    assert torch.equal(y, y_fused)
    out = ops.moe_unpermute(y, inv, w).float().cpu().numpy()
    # routing oracle: the torch definition
    p = torch.softmax(logits.float(), -1)
    rw, ridx = torch.topk(p, K_MOE)
    rw = rw / rw.sum(-1, keepdim=True)
    assert torch.equal(idx.cpu().to(torch.int64), ridx)
    assert torch.allclose(w.cpu(), rw, rtol=1e-5, atol=1e-7)
    counts = torch.bincount(ridx.reshape(-1), minlength=E_MOE)
    assert torch.equal(offs.cpu()[1:].to(torch.int64), torch.cumsum(counts, 0))
    rng = np.random.default_rng(tokens)
    sample = np.unique(np.concatenate([[0, tokens - 1], rng.integers(0, tokens, 30)]))[:32]
    hb = bits_of(hidden)
    worst = 0.0
    for t in sample:
        acc = np.zeros(H_MOE, dtype=np.float32)
        for s in range(K_MOE):       # the combine: fp32 fused multiply-adds in slot order
            ye = oracle_expert(base, int(ridx[t, s]), hb[t])
            acc = np.float32(rw[t, s].item()) * ye + acc
        ref = bf16_round(acc)
        worst = max(worst, float(np.abs(out[t] - ref).max() / np.abs(ref).max()))
    # 1e-3 of the GEMMs, through two bf16 roundings between the projections and one at the end
    assert worst <= 1e-3 + 3 * 2.0 ** -8, (tokens, worst)


# ------------------------------------------------------------------------------------------
# NVFP4 grouped GEMM at 8 experts x 14336 x 4096
# ------------------------------------------------------------------------------------------
def nvfp4_dequant_rows(codes, scales_f32, scale2):
    """codes uint8 [R, K/2], group scales float32 [R, K/16] (e4m3 values), per-tensor scale."""
    return Q.dequantize_nvfp4(codes, scales_f32, scale2).astype(np.float64)


def e4m3_bytes_to_f32(b):
    return torch.from_numpy(np.ascontiguousarray(b)).view(torch.float8_e4m3fn).float().numpy()


def unswizzle_scales(sf_bytes, rows, K):
    """Row-major [rows, K/16] view of an Sm1xx-interleaved scale-factor buffer of one problem
    (128-row x 4-group atoms; the layout the quantizers write and the GEMM reads)."""
    kg = K // 16
    rp = (rows + 127) // 128 * 128
    a = np.asarray(sf_bytes[: rp * kg]).reshape(rp // 128, kg // 4, 32, 4, 4)
    # element (tile m, tile k, r % 32, r // 32 % 4, g % 4)
    out = a.transpose(0, 3, 2, 1, 4).reshape(rp, kg)
    return out[:rows]


@pytest.mark.parametrize("which", ["gate", "down"])
def test_nvfp4_grouped_gemm_8x14336x4096_sampled_vs_dequant_matmul(ops, which):
    E, k, H, I, tokens = 8, 2, 4096, 14336, 4096
    N, K = (I, H) if which == "gate" else (H, I)
    rows = tokens * k
    per = rows // E
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(4)
    codes, sfs, alphas, w_deq_rows = [], [], [], {}
    rng = np.random.default_rng(1)
    cols = np.unique(np.concatenate([[0, N - 1, 127, 128], rng.integers(0, N, 28)]))
    for e in range(E):
        wt = (torch.randn((N, K), generator=g, device=dev) * 0.02).to(torch.bfloat16)
        s2 = max(float(wt.float().abs().max().item()) / 6.0, 1e-12)
        scaled = (wt.float() / s2).to(torch.bfloat16)
        c, sf = ops.bf16_to_nvfp4(scaled)
        codes.append(c)
        sfs.append(sf)
        alphas.append(s2)
        # dequantized sample columns of this expert, from the packed bytes the GEMM reads
        sf_rm = unswizzle_scales(sf.cpu().numpy().reshape(-1), N, K)
        w_deq_rows[e] = nvfp4_dequant_rows(c.cpu().numpy()[cols], e4m3_bytes_to_f32(sf_rm[cols]), s2)
        del wt, scaled
    B = torch.stack(codes)
    SB = torch.stack(sfs)
    al = torch.tensor(alphas, dtype=torch.float32, device=dev)
    x = torch.randn(rows, K, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16).to(dev)
    offs = (torch.arange(E + 1, dtype=torch.int32) * per).to(dev)
    xa, xs, sfo = ops.bf16_to_nvfp4_grouped(x, offs)
    sizes = torch.tensor([[per, N, K]] * E, dtype=torch.int32, device=dev)
    D = torch.empty((rows, N), dtype=torch.bfloat16, device=dev)
    ops.nvfp4_grouped_gemm(xa, B, D, xs, SB, al, offs, sfo, sizes, N, K, "bf16")
    got = D.float().cpu().numpy()
    xa_h, xs_h, sfo_h = xa.cpu().numpy(), xs.cpu().numpy(), sfo.cpu().numpy()
    worst = 0.0
    for e in range(E):
        r_local = np.unique(np.concatenate([[0, per - 1], rng.integers(0, per, 6)]))
        sf_rm = unswizzle_scales(xs_h[int(sfo_h[e]) * (K // 16):], per, K)
        x_deq = nvfp4_dequant_rows(xa_h[e * per + r_local], e4m3_bytes_to_f32(sf_rm[r_local]), 1.0)
        ref = x_deq @ w_deq_rows[e].T
        blk = got[np.ix_(e * per + r_local, cols)]
        worst = max(worst, float(np.abs(blk - ref).max() / np.abs(ref).max()))
    assert worst <= 2e-2, (which, worst)
