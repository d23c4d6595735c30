"""CPU oracle (test infrastructure): ctypes loader for oracle/liblsg_oracle.so.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liblsg_oracle.so")


def build(force=False):
    """Compiles the C restatement with gcc (seconds)."""
    srcs = [os.path.join(_HERE, n) for n in ("lsg_oracle.c", "lsg_oracle_quant.c", "Makefile")]
    if (not force and os.path.exists(LIB_PATH)
            and all(os.path.getmtime(LIB_PATH) >= os.path.getmtime(s) for s in srcs)):
        return LIB_PATH
    subprocess.run(["make", "-C", _HERE, "-B", "liblsg_oracle.so"], check=True,
                   capture_output=True)
    return LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.oracle_f16_to_f32.restype = ctypes.c_float
        _lib.oracle_f16_to_f32.argtypes = [ctypes.c_uint16]
        _lib.oracle_f32_to_f16.restype = ctypes.c_uint16
        _lib.oracle_f32_to_f16.argtypes = [ctypes.c_float]
    return _lib


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _u8(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint8
    return a


def block_values(t):
    return lib().oracle_block_values(int(t))


def block_bytes(t):
    return lib().oracle_block_bytes(int(t))


def quantize_q8_1(x_bf16_bits):
    """x_bf16_bits: uint16 [M,K] (raw bf16).  Returns uint8 [M, K/32, 36]."""
    x = np.ascontiguousarray(x_bf16_bits, dtype=np.uint16)
    M, K = x.shape
    out = np.zeros((M, K // 32, 36), dtype=np.uint8)
    lib().oracle_quantize_q8_1(_ptr(x), _ptr(out), ctypes.c_int(M), ctypes.c_int(K))
    return out


def dequant(t, packed):
    """packed: uint8 [N, row_bytes].  Returns float32 [N, K]."""
    p = _u8(packed)
    N = p.shape[0]
    nblk = p.shape[1] // block_bytes(t)
    out = np.zeros((N, nblk * block_values(t)), dtype=np.float32)
    lib().oracle_dequant_blocks(ctypes.c_int(int(t)), _ptr(p), ctypes.c_long(N * nblk), _ptr(out))
    return out


def mmvq(t, xq, W, K):
    """Integer mat-vec in double precision.  xq uint8 [M,K/32,36]; W uint8 [N,row_bytes]."""
    xq = _u8(xq)
    W = _u8(W)
    M, N = xq.shape[0], W.shape[0]
    out = np.zeros((M, N), dtype=np.float64)
    lib().oracle_mmvq(ctypes.c_int(int(t)), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
                      _ptr(xq), _ptr(W), _ptr(out))
    return out


def dequant_gemm(t, a_bf16_bits, W, K):
    a = np.ascontiguousarray(a_bf16_bits, dtype=np.uint16)
    W = _u8(W)
    M, N = a.shape[0], W.shape[0]
    out = np.zeros((M, N), dtype=np.float64)
    lib().oracle_dequant_gemm(ctypes.c_int(int(t)), ctypes.c_int(M), ctypes.c_int(N),
                              ctypes.c_int(K), _ptr(a), _ptr(W), _ptr(out))
    return out


# ---------------------------------------------------------------------------
# FP8 (e4m3) block-scaled GEMM family, numpy restatements
# ---------------------------------------------------------------------------
def weight_fp8_quant(w_f32):
    """bf16-valued weight [N,K] (as float32) -> (e4m3 bytes [N,K], fp32 scales [NB,KB]).

    Restates weight_fp8_quant_kernel, csrc/smxx/quant/weight_fp8_quant.cu:51-138: one scale
    per 128 x 128 tile = tile amax / 448 (1 for an all-zero tile), values
    clamp(x * (1/scale), +-448) rounded to e4m3; scales[nb, kb] is the K-major buffer
    scales[kb + nb*KB] the GEMM consumes."""
    w = np.asarray(w_f32, dtype=np.float32)
    N, K = w.shape
    NB, KB = (N + 127) // 128, (K + 127) // 128
    q = np.zeros((N, K), np.uint8)
    s = np.zeros((NB, KB), np.float32)
    for nb in range(NB):
        for kb in range(KB):
            tile = w[nb * 128:nb * 128 + 128, kb * 128:kb * 128 + 128]
            amax = np.float32(np.abs(tile).max())
            sc = np.float32(amax / np.float32(448.0)) if amax > 0 else np.float32(1.0)
            inv = np.float32(1.0) / sc
            s[nb, kb] = sc
            scaled = np.clip((tile * inv).astype(np.float32), -448.0, 448.0)
            q[nb * 128:nb * 128 + 128, kb * 128:kb * 128 + 128] = f32_to_e4m3(scaled).reshape(scaled.shape)
    return q, s


def fp8_gemm(a_e4m3, scale_a_mmajor, b_e4m3, scale_b, M, N, K):
    """Block-scaled e4m3 GEMM in float64: the operand contract of launch_fp8_gemm,
    csrc/sm120/gemm/fp8/fp8_gemm.h:18-44:
      D[m,n] = sum_kb scale_A[m + kb*M] * scale_B[kb + (n/128)*KB] * sum_{k in kb} A[m,k]*B[n,k]."""
    a = e4m3_to_f32(np.asarray(a_e4m3, dtype=np.uint8)).astype(np.float64).reshape(M, K)
    b = e4m3_to_f32(np.asarray(b_e4m3, dtype=np.uint8)).astype(np.float64).reshape(N, K)
    KB = (K + 127) // 128
    sa = np.asarray(scale_a_mmajor, dtype=np.float64).reshape(KB, M)    # [kb, m]
    sb = np.asarray(scale_b, dtype=np.float64).reshape(-1, KB)          # [nb, kb]
    out = np.zeros((M, N))
    for kb in range(KB):
        ks = slice(kb * 128, min(K, kb * 128 + 128))
        out += (a[:, ks] @ b[:, ks].T) * sa[kb][:, None] * np.repeat(sb[:, kb], 128)[:N][None, :]
    return out


# ---------------------------------------------------------------------------
# The reference's own CUDA kernels, compiled for sm_100a from its sources where they
# lie (oracle/Makefile target `ref`).  Optional second checker for the GPU tests.
# ---------------------------------------------------------------------------
REF_LIB_PATH = os.path.join(_HERE, "_ref", "libref_gguf.so")
_ref = None


def ref_lib():
    """ctypes handle of oracle/_ref/libref_gguf.so, or None when it has not been built."""
    global _ref
    if _ref is None and os.path.exists(REF_LIB_PATH):
        try:
            _ref = ctypes.CDLL(REF_LIB_PATH)
        except OSError:
            _ref = None
    return _ref


REF_GROUPED_LIB_PATH = os.path.join(_HERE, "_ref", "libref_grouped.so")
_ref_grouped = None


def ref_grouped_lib():
    """ctypes handle of oracle/_ref/libref_grouped.so (the reference's grouped GGUF launchers,
    its routing-metadata kernels, its mma.sync prefill GEMM and its FP8 weight quantizer), or
    None when it has not been built (it needs CuTe headers, see oracle/Makefile)."""
    global _ref_grouped
    if _ref_grouped is None and os.path.exists(REF_GROUPED_LIB_PATH):
        try:
            _ref_grouped = ctypes.CDLL(REF_GROUPED_LIB_PATH)
            _ref_grouped.ref_gguf_grouped_gemm_workspace_bytes.restype = ctypes.c_size_t
        except OSError:
            _ref_grouped = None
    return _ref_grouped


# ---------------------------------------------------------------------------
# FP8 / NVFP4 activation quantizers
# ---------------------------------------------------------------------------
def f32_to_e4m3(values):
    L = lib()
    L.oracle_f32_to_e4m3.restype = ctypes.c_uint8
    L.oracle_f32_to_e4m3.argtypes = [ctypes.c_float]
    v = np.asarray(values, dtype=np.float32).ravel()
    return np.array([L.oracle_f32_to_e4m3(float(x)) for x in v], dtype=np.uint8)


def e4m3_to_f32(bits):
    L = lib()
    L.oracle_e4m3_to_f32.restype = ctypes.c_float
    L.oracle_e4m3_to_f32.argtypes = [ctypes.c_uint8]
    return np.array([L.oracle_e4m3_to_f32(int(b)) for b in np.asarray(bits).ravel()], dtype=np.float32)


def dynamic_fp8_quant(x_bf16_bits, m_major=False):
    """Returns (e4m3 bytes [M,K], fp32 scales [M,nb] or [nb,M])."""
    x = np.ascontiguousarray(x_bf16_bits, dtype=np.uint16)
    M, K = x.shape
    nb = (K + 127) // 128
    out = np.zeros((M, K), dtype=np.uint8)
    scales = np.zeros((nb, M) if m_major else (M, nb), dtype=np.float32)
    lib().oracle_dynamic_fp8_quant(_ptr(x), _ptr(out), _ptr(scales), ctypes.c_int(M),
                                   ctypes.c_int(K), ctypes.c_int(1 if m_major else 0))
    return out, scales


def nvfp4_sf_offsets(expert_offsets):
    offs = np.ascontiguousarray(expert_offsets, dtype=np.int32)
    E = offs.shape[0] - 1
    sf = np.zeros(E + 1, dtype=np.int32)
    lib().oracle_nvfp4_sf_offsets(_ptr(offs), _ptr(sf), ctypes.c_int(E))
    return sf


def bf16_to_nvfp4_grouped(x_bf16_bits, expert_offsets, input_scales=None):
    """Returns (packed [T,K/2], scales [padded_total*K/16], sf_offsets [E+1])."""
    x = np.ascontiguousarray(x_bf16_bits, dtype=np.uint16)
    T, K = x.shape
    offs = np.ascontiguousarray(expert_offsets, dtype=np.int32)
    E = offs.shape[0] - 1
    sf = nvfp4_sf_offsets(offs)
    packed = np.zeros((T, K // 2), dtype=np.uint8)
    scales = np.zeros(int(sf[E]) * (K // 16), dtype=np.uint8)
    isc = None
    if input_scales is not None:
        isc = np.ascontiguousarray(input_scales, dtype=np.float32)
    lib().oracle_bf16_to_nvfp4_grouped(_ptr(x), _ptr(packed), _ptr(scales), _ptr(offs), _ptr(sf),
                                       _ptr(isc) if isc is not None else None,
                                       ctypes.c_int(T), ctypes.c_int(E), ctypes.c_int(K))
    return packed, scales, sf
