"""CPU tests: the oracle against the reference's golden vectors and known answers."""
import os

import numpy as np
import pytest

import oracle
from layerstormgemmkernels_b200 import quantize as Q
from layerstormgemmkernels_b200.capi import GGUF_TYPES, BLOCK_BYTES, BLOCK_VALUES

T = GGUF_TYPES


def bf16_bits(x):
    """float32 array -> raw bf16 (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def bf16_to_f32(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


@pytest.fixture(scope="module")
def q4k(golden_dir):
    return np.load(os.path.join(golden_dir, "q4k_reference.npz"))


def test_block_sizes_match_reference_table():
    # tests/test_gguf_grouped_gemm.py:49-59 (GGUF_SPEC) and gguf_dequant_gemm.cu:292-307
    spec = {"Q2_K": (0, 84, 256), "Q3_K": (1, 110, 256), "Q4_K": (2, 144, 256),
            "Q5_K": (3, 176, 256), "Q6_K": (4, 210, 256), "Q8_0": (5, 34, 32),
            "MXFP4": (6, 17, 32)}
    for name, (t, b, v) in spec.items():
        assert T[name] == t
        assert oracle.block_bytes(t) == b == BLOCK_BYTES[t]
        assert oracle.block_values(t) == v == BLOCK_VALUES[t]
    assert oracle.block_bytes(T["Q4_0"]) == 18 and oracle.block_values(T["Q4_0"]) == 32


def test_q4k_dequant_matches_reference_python(q4k):
    got = oracle.dequant(T["Q4_K"], q4k["packed"])
    # ref_q4k_dequant (tests/test_reference.py:284-323) computes d*sc*q - dmin*m in fp32
    np.testing.assert_allclose(got, q4k["dequant"], rtol=0, atol=1e-7)


def test_q4k_dequant_gemm_matches_reference_python(q4k):
    got = oracle.dequant_gemm(T["Q4_K"], q4k["x_bf16"], q4k["packed"], 512)
    ref = q4k["gemm"].astype(np.float64)
    assert np.abs(got - ref).max() <= 1e-5 * np.abs(ref).max()


def test_q4k_scale_packing_known_answers(q4k):
    # tests/test_reference.py:545-557
    for sc, mn, packed in ((q4k["ka_sc"], q4k["ka_mn"], q4k["ka_packed"]),
                           (q4k["ka_sc2"], q4k["ka_mn2"], q4k["ka_packed2"])):
        np.testing.assert_array_equal(Q.pack_k4_scales(sc, mn), packed)
        # decode through the oracle: a block whose quants are all 1 and d = dmin = 1
        blk = np.zeros((1, 144), dtype=np.uint8)
        blk[0, 0:2] = np.frombuffer(np.float16(1.0).tobytes(), dtype=np.uint8)
        blk[0, 2:4] = np.frombuffer(np.float16(1.0).tobytes(), dtype=np.uint8)
        blk[0, 4:16] = packed
        blk[0, 16:] = 0x11
        out = oracle.dequant(T["Q4_K"], blk).reshape(8, 32)
        np.testing.assert_array_equal(out[:, 0], sc.astype(np.float32) - mn.astype(np.float32))


def test_q4k_known_block():
    # tests/test_reference.py:559-577: d=1, dmin=.5, scales=mins=1, quants=7 -> 6.5
    blk = np.zeros((1, 144), dtype=np.uint8)
    blk[0, 0:2] = np.frombuffer(np.float16(1.0).tobytes(), dtype=np.uint8)
    blk[0, 2:4] = np.frombuffer(np.float16(0.5).tobytes(), dtype=np.uint8)
    blk[0, 4:16] = Q.pack_k4_scales(np.ones(8, np.uint8), np.ones(8, np.uint8))
    blk[0, 16:] = 0x77
    np.testing.assert_array_equal(oracle.dequant(T["Q4_K"], blk), np.full((1, 256), 6.5, np.float32))


def test_host_q4k_packer_is_byte_identical_to_reference(q4k):
    np.testing.assert_array_equal(Q.quantize_q4_k(q4k["w"]), q4k["packed"])


def _mxfp4_numpy_reference(raw, K):
    """Independent MXFP4 decode, written from the OCP MX definition."""
    table = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float32)
    N = raw.shape[0]
    b = raw.reshape(N, K // 32, 17)
    e = b[:, :, 0].astype(np.int32)
    scale = np.ldexp(np.float32(1.0), e - 127).astype(np.float32)
    lo = table[b[:, :, 1:] & 0xF]
    hi = table[b[:, :, 1:] >> 4]
    return (np.concatenate([lo, hi], -1) * scale[..., None]).reshape(N, K)


def test_mxfp4_decode_against_independent_reference():
    raw = Q.random_gguf_weight("MXFP4", 8, 128, seed=3)
    raw.reshape(8, 4, 17)[:, 0, 0] = 127   # scale 1
    raw.reshape(8, 4, 17)[:, 1, 0] = 1     # denormal half-scale path
    got = oracle.dequant(T["MXFP4"], raw)
    np.testing.assert_allclose(got, _mxfp4_numpy_reference(raw, 128), rtol=0, atol=1e-6)


@pytest.mark.parametrize("name", ["Q6_K", "Q8_0", "Q4_0"])
def test_host_packers_roundtrip(name):
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((16, 512)) * 0.02).astype(np.float32)
    deq = oracle.dequant(T[name], Q.QUANTIZERS[name](w))
    cos = (w * deq).sum() / np.sqrt((w * w).sum() * (deq * deq).sum())
    assert cos > {"Q6_K": 0.999, "Q8_0": 0.9999, "Q4_0": 0.99}[name]


@pytest.mark.parametrize("name", list(T))
def test_int_form_equals_dequant(name):
    """w = A*Q + B (gguf_int_policy.h) must reproduce dequant_*_block value by value:
    mmvq with one-hot unit activations reads the weight back."""
    t = T[name]
    K = 2 * BLOCK_VALUES[t] if BLOCK_VALUES[t] == 256 else 256
    W = Q.random_gguf_weight(name, 4, K, seed=11)
    deq = oracle.dequant(t, W)
    # activation row k = 127 * e_k  ->  Q8_1: d = 1, q = 127 at k
    x = np.zeros((K, K), dtype=np.float32)
    np.fill_diagonal(x, 127.0)
    xq = oracle.quantize_q8_1(bf16_bits(x))
    y = oracle.mmvq(t, xq, W, K)          # [K, 4] = 127 * W^T
    np.testing.assert_allclose(y.T / 127.0, deq, rtol=2e-6, atol=1e-7)


def test_q8_1_quantizer_properties():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 256)).astype(np.float32)
    x[1, 32:64] = 0.0
    bits = bf16_bits(x)
    xb = bf16_to_f32(bits)
    blocks = oracle.quantize_q8_1(bits)
    d = blocks[:, :, 0:2].copy().view(np.float16).astype(np.float32)[..., 0]
    s = blocks[:, :, 2:4].copy().view(np.float16).astype(np.float32)[..., 0]
    q = blocks[:, :, 4:].view(np.int8).astype(np.float32)
    g = xb.reshape(3, 8, 32)
    amax = np.abs(g).max(-1)
    np.testing.assert_array_equal(d, (amax / np.float32(127.0)).astype(np.float16).astype(np.float32))
    assert np.abs(q).max() == 127 and (q[1, 1] == 0).all() and d[1, 1] == 0
    np.testing.assert_allclose(s, g.sum(-1), rtol=2e-3, atol=1e-3)
    dd = (amax / np.float32(127.0))[..., None]
    with np.errstate(divide="ignore", invalid="ignore"):
        np.testing.assert_array_equal(q, np.where(dd > 0, np.rint(g / dd), 0))


def test_fp16_conversions_are_exact():
    L = oracle.lib()
    rng = np.random.default_rng(1)
    vals = np.concatenate([rng.standard_normal(3000).astype(np.float32) * s
                           for s in (1e-8, 6e-8, 1e-5, 1.0, 1000.0)])
    got = np.array([L.oracle_f32_to_f16(float(v)) for v in vals], dtype=np.uint16)
    np.testing.assert_array_equal(got, vals.astype(np.float16).view(np.uint16))
