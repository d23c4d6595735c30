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
