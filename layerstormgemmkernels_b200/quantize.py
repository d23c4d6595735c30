"""Host-side (numpy) GGUF weight packers used to make inputs for tests and benchmarks.

These run offline, once per weight; they are not on the hot path.

* quantize_q4_k restates, vectorised, the rule of the reference's pure-Python
  packer quantize_to_q4k (tests/test_reference.py:334-432: per-32 min/max scale,
  6-bit scale/min against the super-block maxima, re-quantisation against the
  rounded scales) and produces the same bytes.
* The reference has no packers for the other types; their rules are the simple
  ones written in each docstring.
* random_gguf_weight restates make_gguf_weight
  (tests/test_gguf_grouped_gemm.py:66-83): random bytes with finite scale fields.
"""
import numpy as np

from .formats import BLOCK_BYTES, BLOCK_VALUES, GGUF_TYPES, Q4_K, Q6_K, Q8_0, Q4_0  # noqa: F401


def _f16_bytes(x):
    """float array [...] -> uint8 [..., 2] little-endian fp16."""
    return np.ascontiguousarray(x.astype(np.float16)).view(np.uint8).reshape(*x.shape, 2)


def pack_k4_scales(sc, mn):
    """6-bit scales/mins [..., 8] uint8 -> the 12-byte Q4_K/Q5_K field [..., 12]."""
    sc = sc.astype(np.uint8) & 63
    mn = mn.astype(np.uint8) & 63
    out = np.zeros(sc.shape[:-1] + (12,), dtype=np.uint8)
    out[..., 0:4] = sc[..., 0:4] | ((sc[..., 4:8] >> 4) << 6)
    out[..., 4:8] = mn[..., 0:4] | ((mn[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 0x0F) | ((mn[..., 4:8] & 0x0F) << 4)
    return out


def quantize_q4_k(w):
    """float [N,K] -> uint8 [N, K/256*144] Q4_K blocks."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    N, K = w.shape
    assert K % 256 == 0
    nb = K // 256
    sub = w.reshape(N, nb, 8, 32)
    vmin = sub.min(-1)
    vmax = sub.max(-1)
    min_off = np.maximum(np.float32(0), -vmin).astype(np.float32)
    rng = (vmax + min_off).astype(np.float32)
    # python-float arithmetic in the reference: range/15.0 is done in double
    scale = np.where(rng < 1e-15, 0.0, rng.astype(np.float64) / 15.0)
    scales = scale.astype(np.float32)          # stored into a float32 array there
    mins = min_off.astype(np.float32)
    max_scale = scales.max(-1).astype(np.float64)
    max_min = mins.max(-1).astype(np.float64)
    with np.errstate(divide="ignore", invalid="ignore"):
        d = np.where(max_scale > 0, max_scale / 63.0, 0.0)
        dmin = np.where(max_min > 0, max_min / 63.0, 0.0)
        inv_scale = np.where(max_scale > 0, 63.0 / max_scale, 0.0)
        inv_min = np.where(max_min > 0, 63.0 / max_min, 0.0)
    sc_q = np.clip(np.round(inv_scale[..., None] * scales), 0, 63).astype(np.uint8)
    mn_q = np.clip(np.round(inv_min[..., None] * mins), 0, 63).astype(np.uint8)
    d16 = d.astype(np.float16).astype(np.float32)
    dmin16 = dmin.astype(np.float16).astype(np.float32)
    d_j = d16[..., None] * sc_q.astype(np.float32)
    dm_j = dmin16[..., None] * mn_q.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.round((sub + dm_j[..., None]) / d_j[..., None])
    q = np.where(d_j[..., None] == 0, 0, np.clip(q, 0, 15)).astype(np.uint8)
    out = np.zeros((N, nb, 144), dtype=np.uint8)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:4] = _f16_bytes(dmin)
    out[..., 4:16] = pack_k4_scales(sc_q, mn_q)
    lo = q[:, :, 0::2, :]   # sub-blocks 0,2,4,6 -> low nibbles of pairs 0..3
    hi = q[:, :, 1::2, :]
    out[..., 16:144] = ((lo & 0x0F) | ((hi & 0x0F) << 4)).reshape(N, nb, 128)
    return out.reshape(N, nb * 144)


def quantize_q6_k(w):
    """float [N,K] -> Q6_K blocks (210 B / 256 values).

    Rule: per 16 values s = maxabs/32; d = max|s|/127 (fp16); int8 scale = rn(s/d);
    q = clamp(rn(x / (d*scale)) + 32, 0, 63).  Layout as ggml block_q6_K.
    """
    w = np.ascontiguousarray(w, dtype=np.float32)
    N, K = w.shape
    assert K % 256 == 0
    nb = K // 256
    g = w.reshape(N, nb, 16, 16)
    s = np.abs(g).max(-1) / np.float32(32.0)
    d = (s.max(-1) / np.float32(127.0)).astype(np.float16).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(d[..., None] > 0, np.round(s / d[..., None]), 0)
    sc = np.clip(sc, -128, 127).astype(np.int8)
    eff = d[..., None] * sc.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(eff[..., None] != 0, np.round(g / eff[..., None]), 0)
    q = (np.clip(q, -32, 31) + 32).astype(np.uint8).reshape(N, nb, 256)
    out = np.zeros((N, nb, 210), dtype=np.uint8)
    # value index 128*ip + 32*quad + il  <->  ql[64ip + 32(quad&1) + il] nibble (quad>>1),
    # qh[32ip + il] bits 2*quad..2*quad+1
    v = q.reshape(N, nb, 2, 4, 32)  # [ip][quad][il]
    lo4 = v & 0x0F
    hi2 = v >> 4
    ql = np.zeros((N, nb, 2, 64), dtype=np.uint8)
    ql[..., 0:32] = lo4[:, :, :, 0, :] | (lo4[:, :, :, 2, :] << 4)
    ql[..., 32:64] = lo4[:, :, :, 1, :] | (lo4[:, :, :, 3, :] << 4)
    qh = (hi2[:, :, :, 0, :] | (hi2[:, :, :, 1, :] << 2) | (hi2[:, :, :, 2, :] << 4)
          | (hi2[:, :, :, 3, :] << 6)).astype(np.uint8)
    out[..., 0:128] = ql.reshape(N, nb, 128)
    out[..., 128:192] = qh.reshape(N, nb, 64)
    out[..., 192:208] = sc.view(np.uint8)
    out[..., 208:210] = _f16_bytes(d)
    return out.reshape(N, nb * 210)


def quantize_q8_0(w):
    """float [N,K] -> Q8_0 blocks (34 B / 32): d = maxabs/127 (fp16), q = rn(x/d)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    N, K = w.shape
    assert K % 32 == 0
    nb = K // 32
    g = w.reshape(N, nb, 32)
    d = (np.abs(g).max(-1) / np.float32(127.0)).astype(np.float16)
    d32 = d.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(d32[..., None] > 0, np.round(g / d32[..., None]), 0)
    q = np.clip(q, -127, 127).astype(np.int8)
    out = np.zeros((N, nb, 34), dtype=np.uint8)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:34] = q.view(np.uint8)
    return out.reshape(N, nb * 34)


def quantize_q4_0(w):
    """float [N,K] -> Q4_0 blocks (18 B / 32), the ggml rule: d = (signed value of
    largest magnitude) / -8 as fp16, q = clamp(rn(x/d) + 8, 0, 15); low nibble holds
    value j, high nibble value j+16."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    N, K = w.shape
    assert K % 32 == 0
    nb = K // 32
    g = w.reshape(N, nb, 32)
    idx = np.abs(g).argmax(-1)
    smax = np.take_along_axis(g, idx[..., None], -1)[..., 0]
    d = (smax / np.float32(-8.0)).astype(np.float16)
    d32 = d.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(d32[..., None] != 0, np.round(g / d32[..., None]), 0)
    q = np.clip(q + 8, 0, 15).astype(np.uint8)
    out = np.zeros((N, nb, 18), dtype=np.uint8)
    out[..., 0:2] = _f16_bytes(d)
    out[..., 2:18] = q[..., 0:16] | (q[..., 16:32] << 4)
    return out.reshape(N, nb * 18)


QUANTIZERS = {"Q4_K": quantize_q4_k, "Q6_K": quantize_q6_k, "Q8_0": quantize_q8_0,
              "Q4_0": quantize_q4_0}

# (byte offset, value) of every fp16 scale field, so that random bytes never
# decode to Inf/NaN; E8M0 exponent byte for MXFP4.
_SCALE_FIELDS = {
    "Q2_K": [(80, 0.04), (82, 0.02)], "Q3_K": [(108, 0.012)], "Q4_K": [(0, 0.02), (2, 0.01)],
    "Q5_K": [(0, 0.015), (2, 0.008)], "Q6_K": [(208, 0.004)], "Q8_0": [(0, 0.02)],
    "Q4_0": [(0, 0.02)], "MXFP4": [],
}


def random_gguf_weight(name, N, K, seed):
    """Random valid-layout packed weight, uint8 [N, K/QK*bytes]."""
    t = GGUF_TYPES[name]
    bb, qk = BLOCK_BYTES[t], BLOCK_VALUES[t]
    nb = K // qk
    rng = np.random.default_rng(seed)
    w = rng.integers(0, 256, size=(N, nb, bb), dtype=np.uint8)
    for off, val in _SCALE_FIELDS[name]:
        w[:, :, off:off + 2] = np.frombuffer(np.float16(val).tobytes(), dtype=np.uint8)
    if name == "MXFP4":
        w[:, :, 0] = 121
    return w.reshape(N, nb * bb)


E2M1_TABLE = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                       -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32)


def _to_e4m3_f32(x):
    """float32 array -> nearest e4m3 value as float32 (torch's float8_e4m3fn rounding)."""
    import torch
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(torch.float8_e4m3fn).float().numpy()


def quantize_nvfp4(w):
    """float [N,K] -> (uint8 [N,K/2] codes, float32 [N,K/16] e4m3-valued group scales,
    float32 global scale).  Restates the reference's quantize_to_nvfp4
    (tests/test_reference.py:162-199): global scale amax/6, group scale
    amax_g/(6*global) rounded to e4m3, nearest table entry (first on ties)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    N, K = w.shape
    assert K % 16 == 0
    scale2 = np.float32(max(np.abs(w).max() / np.float32(6.0), np.float32(1e-12)))
    g = w.reshape(N, K // 16, 16)
    raw = np.abs(g).max(-1) / (scale2 * np.float32(6.0))
    raw = np.clip(raw, np.float32(1e-12), np.float32(448.0)).astype(np.float32)
    sc = np.maximum(_to_e4m3_f32(raw), np.float32(1e-12)).astype(np.float32)
    local = w / (np.repeat(sc, 16, axis=1) * scale2)
    idx = np.abs(local[..., None] - E2M1_TABLE).argmin(-1).astype(np.uint8)
    pairs = idx.reshape(N, K // 2, 2)
    return (pairs[:, :, 0] | (pairs[:, :, 1] << 4)).astype(np.uint8), sc, scale2


def dequantize_nvfp4(codes_u8, scales, scale2=1.0):
    """Inverse of quantize_nvfp4 (reference: ref_nvfp4_dequant, tests/test_reference.py:107-128)."""
    N, half = codes_u8.shape
    idx = np.stack([codes_u8 & 0xF, codes_u8 >> 4], -1).reshape(N, half * 2)
    return E2M1_TABLE[idx] * np.repeat(np.asarray(scales, np.float32), 16, axis=1) * np.float32(scale2)
