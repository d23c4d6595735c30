"""CPU tests: FP8 / NVFP4 quantizer oracles against the reference's Python definitions."""
import os

import numpy as np
import pytest
import torch

import oracle
from test_oracle import bf16_bits, bf16_to_f32

E2M1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float32)


def test_e4m3_conversion_matches_torch_everywhere():
    rng = np.random.default_rng(0)
    v = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s
                        for s in (1e-4, 1e-3, 1e-2, .1, 1, 10, 100, 300)])
    v = np.clip(v, -448, 448)
    got = oracle.f32_to_e4m3(v)
    want = torch.from_numpy(v).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    np.testing.assert_array_equal(got, want)
    # saturation above the largest finite value, ties at the top
    np.testing.assert_array_equal(oracle.f32_to_e4m3([448, 463.9, 464, 480, 1e9, -1e9]),
                                  [0x7E, 0x7E, 0x7E, 0x7E, 0x7E, 0xFE])
    allb = np.arange(256, dtype=np.uint8)
    f = oracle.e4m3_to_f32(allb)
    ft = torch.from_numpy(allb).view(torch.float8_e4m3fn).float().numpy()
    assert ((f == ft) | (np.isnan(f) & np.isnan(ft))).all()


def test_fp8_quant_matches_reference_python(golden_dir):
    # ref_dynamic_fp8_quant (tests/test_reference.py:56-73) returns the scaled, clamped,
    # UN-rounded values and the scales
    z = np.load(os.path.join(golden_dir, "fp8_reference.npz"))
    out, sc = oracle.dynamic_fp8_quant(z["x_bf16"])
    np.testing.assert_array_equal(sc, z["scales"])
    deq = oracle.e4m3_to_f32(out).reshape(out.shape)
    ref = z["scaled"]
    # e4m3 has 3 mantissa bits: rounding error <= 2^-4 relative (half an ulp), 2^-10 absolute
    assert (np.abs(deq - ref) <= np.maximum(np.abs(ref) * 2.0 ** -4, 2.0 ** -10) + 1e-7).all()
    # all-zero block -> scale 1.0, codes 0
    assert sc[2, 1] == 1.0 and (out[2, 128:256] == 0).all()
    out_m, sc_m = oracle.dynamic_fp8_quant(z["x_bf16"], m_major=True)
    np.testing.assert_array_equal(out_m, out)
    np.testing.assert_array_equal(sc_m, sc.T)


def test_nvfp4_table_matches_reference(golden_dir):
    z = np.load(os.path.join(golden_dir, "nvfp4_reference.npz"))
    np.testing.assert_array_equal(z["table"], E2M1)


def _decode_grouped(packed, scales, sf, offs, K):
    """Decode with the layout helper the reference's tests use (tests/test_kernels.py:100-126)."""
    T = packed.shape[0]
    gpr = K // 16
    lo, hi = packed & 0xF, packed >> 4
    codes = np.stack([lo, hi], -1).reshape(T, K)
    vals = E2M1[codes]
    sc = np.zeros((T, gpr), np.float32)
    dec = oracle.e4m3_to_f32(np.arange(256, dtype=np.uint8))
    for e in range(len(offs) - 1):
        for r in range(offs[e], offs[e + 1]):
            lr = r - offs[e]
            for g in range(gpr):
                off = ((lr // 128) * ((gpr + 3) // 4) + g // 4) * 512 + (lr % 32) * 16 + ((lr % 128) // 32) * 4 + g % 4
                sc[r, g] = dec[scales[sf[e] * gpr + off]]
    return vals * np.repeat(sc, 16, axis=1)


def test_nvfp4_grouped_quant_roundtrip_and_layout():
    # tests/test_kernels.py:474-497: ragged experts incl. an empty one
    K = 256
    offs = [0, 3, 3, 131, 148]
    rng = np.random.default_rng(21)
    x = (rng.standard_normal((offs[-1], K)) * 0.5).astype(np.float32)
    bits = bf16_bits(x)
    packed, scales, sf = oracle.bf16_to_nvfp4_grouped(bits, offs)
    np.testing.assert_array_equal(sf, [0, 128, 128, 256, 384])
    assert scales.shape[0] == 384 * (K // 16)
    xh = _decode_grouped(packed, scales, sf, offs, K)
    xb = bf16_to_f32(bits)
    for e in range(4):
        s, t = offs[e], offs[e + 1]
        if s == t:
            continue
        a, b = xb[s:t].ravel(), xh[s:t].ravel()
        assert (a * b).sum() / np.sqrt((a * a).sum() * (b * b).sum()) > 0.99
    # padding rows of the scale sections stay zero
    used = np.zeros_like(scales, dtype=bool)
    gpr = K // 16
    for e in range(4):
        for lr in range(offs[e + 1] - offs[e]):
            for g in range(gpr):
                off = ((lr // 128) * (gpr // 4) + g // 4) * 512 + (lr % 32) * 16 + ((lr % 128) // 32) * 4 + g % 4
                used[sf[e] * gpr + off] = True
    assert (scales[~used] == 0).all() and (scales[used] != 0).all()


def test_nvfp4_rounding_ties_go_up_in_magnitude():
    # thresholds .25 .75 1.25 1.75 2.5 3.5 5 are INCLUSIVE (detail header :54-60): with a
    # group scale of exactly 1.0 (amax = 6) the mid-points map to the larger code
    vals = np.array([6, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -5.0, 0.2499, 4.99, 0, 0, 0, 0],
                    np.float32)
    x = np.tile(vals, (1, 4))                       # K = 64
    packed, scales, sf = oracle.bf16_to_nvfp4_grouped(bf16_bits(x), [0, 1])
    codes = np.stack([packed & 0xF, packed >> 4], -1).reshape(1, 64)[0, :16]
    # 0.2499 and 4.99 are not bf16-exact: they become 0.25 (-> code 1) and 5.0 (-> code 7)
    np.testing.assert_array_equal(codes, [7, 1, 2, 3, 4, 5, 6, 7, 9, 15, 1, 7, 0, 0, 0, 0])
    assert oracle.e4m3_to_f32(scales[:1])[0] == 1.0


def test_nvfp4_tiny_values_hit_the_scale_floor_and_input_scales_lift_it():
    # tests/test_kernels.py:499-540
    K = 256
    offs = [0, 64, 128]
    rng = np.random.default_rng(33)
    x = (rng.standard_normal((128, K)) * 1e-3).astype(np.float32)
    bits = bf16_bits(x)
    xb = bf16_to_f32(bits)

    def cos(isc):
        packed, scales, sf = oracle.bf16_to_nvfp4_grouped(bits, offs, isc)
        xh = _decode_grouped(packed, scales, sf, offs, K)
        if isc is not None:
            for e in range(2):
                xh[offs[e]:offs[e + 1]] *= isc[e]
        return (xb * xh).sum() / np.sqrt((xb * xb).sum() * (xh * xh).sum())

    isc = np.array([np.abs(xb[offs[e]:offs[e + 1]]).max() / (448.0 * 6.0) for e in range(2)], np.float32)
    assert cos(isc) > 0.99 and cos(isc) > cos(None)


def test_host_nvfp4_weight_quantizer_matches_reference(golden_dir):
    from layerstormgemmkernels_b200 import quantize as Q
    z = np.load(os.path.join(golden_dir, "nvfp4_reference.npz"))
    codes, sc, s2 = Q.quantize_nvfp4(z["w"])
    np.testing.assert_array_equal(codes, z["w_u8"])
    np.testing.assert_array_equal(sc, z["w_scale"])
    assert s2 == z["w_scale2"]
    deq = Q.dequantize_nvfp4(codes, sc, s2)
    np.testing.assert_allclose(deq, z["dequant"], rtol=1e-6, atol=0)
    np.testing.assert_allclose(z["x"].astype(np.float64) @ deq.astype(np.float64).T, z["gemm"], rtol=0,
                               atol=1e-5 * np.abs(z["gemm"]).max())


def test_fp8_weight_quant_and_gemm_oracle_consistency():
    """The numpy restatements of weight_fp8_quant and of the block-scaled GEMM contract:
    quantize -> GEMM reproduces the fp32 product to e4m3 precision, scales are tile amax / 448,
    an all-zero tile gets scale 1 (csrc/smxx/quant/weight_fp8_quant.cu:102-105)."""
    rng = np.random.default_rng(4)
    N, K, M = 200, 384, 6
    w = (rng.standard_normal((N, K)) * 0.1).astype(np.float32)
    w[128:, 256:] = 0.0
    q, s = oracle.weight_fp8_quant(w)
    assert s.shape == (2, 3) and s[1, 2] == np.float32(1.0)
    assert np.isclose(s[0, 0], np.abs(w[:128, :128]).max() / 448.0)
    deq = (oracle.e4m3_to_f32(q).reshape(N, K).astype(np.float64) *
           np.repeat(np.repeat(s.astype(np.float64), 128, 0)[:N], 128, 1)[:, :K])
    assert np.abs(deq - w).max() <= np.abs(w).max() * 2.0 ** -4
    x = rng.standard_normal((M, K)).astype(np.float32)
    # activations with unit scales and e4m3-representable values
    xa = oracle.f32_to_e4m3(np.clip(x, -448, 448))
    sa = np.ones((3, M), np.float32)
    out = oracle.fp8_gemm(xa, sa, q, s, M, N, K)
    ref = oracle.e4m3_to_f32(xa).reshape(M, K).astype(np.float64) @ deq.T
    assert np.allclose(out, ref, rtol=1e-9, atol=1e-9)
