"""Host-side mirror of the reference's Python operator surface for the GGUF decode path
(csrc/bindings_python.cu of kkontosis/LayerStoRmGemmKernels): same names, argument order,
defaults, checks and error types, implemented over the C ABI of liblsg_b200.so.

torch is used for device memory and the current stream only.  Every operator runs
hand-written sm_100a kernels; nothing here computes on the CPU.
"""
import ctypes

import torch

from . import capi

_lib = capi.lib


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _require(cond, msg):
    # the reference raises through TORCH_CHECK -> RuntimeError
    if not cond:
        raise RuntimeError(msg)


def quantize_q8_1(x):
    """bf16 [M,K] -> uint8 [M, K/32, 36] Q8_1 blocks (d, sum, 32 x int8).

    No Python counterpart in the reference (gguf_quantize_q8_1_cuda is C++ only,
    csrc/sm120/gemm/gguf/gguf_mmvq.cu:124-128); exposed for bit-exactness checks.
    """
    _require(x.is_cuda and x.dtype == torch.bfloat16, "quantize_q8_1: x must be BF16 on CUDA")
    _require(x.dim() == 2 and x.is_contiguous(), "quantize_q8_1: x must be contiguous [M, K]")
    M, K = x.shape
    out = torch.empty((M, K // 32, 36), dtype=torch.uint8, device=x.device)
    capi.check(_lib.lsg_quantize_q8_1(_ptr(x), _ptr(out), M, K, _stream()))
    return out


def _gemm_params(A, B_packed, C, type_i, N, K, out_dtype):
    return capi.GgufMmvqParams(M=A.shape[0], N=int(N), K=int(K), A=A.data_ptr(),
                               B=B_packed.data_ptr(), C=C.data_ptr(), type=int(type_i),
                               out_dtype=out_dtype)


def gguf_mmvq(A, B_packed, type, N, K, out_dtype=torch.bfloat16):
    """GGUF integer mat-vec: bf16 A[M,K] @ decode(B)^T -> [M,N].

    Mirrors gguf_mmvq (csrc/bindings_python.cu:613-643).  out_dtype=torch.float32
    returns the un-rounded accumulator (an extension used by the parity tests).
    """
    _require(A.is_cuda and A.dtype == torch.bfloat16, "gguf_mmvq: A must be BF16 on CUDA")
    _require(A.dim() == 2 and A.is_contiguous(), "gguf_mmvq: A must be contiguous [M, K]")
    _require(A.size(1) == K, "gguf_mmvq: A.size(1) != K")
    _require(B_packed.is_cuda and B_packed.dtype == torch.uint8 and B_packed.is_contiguous(),
             "gguf_mmvq: B_packed must be contiguous uint8 on CUDA")
    _require(out_dtype in (torch.bfloat16, torch.float32), "gguf_mmvq: out_dtype bf16 or f32")
    M = A.size(0)
    C = torch.empty((M, N), dtype=out_dtype, device=A.device)
    ws_bytes = _lib.lsg_gguf_mmvq_workspace_bytes(M, int(K))
    ws = torch.empty((max(ws_bytes, 1),), dtype=torch.uint8, device=A.device)
    p = _gemm_params(A, B_packed, C, type, N, K,
                     capi.DTYPE_F32 if out_dtype == torch.float32 else capi.DTYPE_BF16)
    capi.check(_lib.lsg_gguf_mmvq(ctypes.byref(p), _ptr(ws), ws_bytes, _stream()))
    return C


def gguf_mmvq_q8_1(xq, B_packed, type, N, K, out_dtype=torch.bfloat16):
    """Same mat-vec on pre-quantized activations (uint8 [M, K/32, 36])."""
    _require(xq.is_cuda and xq.dtype == torch.uint8 and xq.is_contiguous(),
             "gguf_mmvq_q8_1: xq must be contiguous uint8 on CUDA")
    M = xq.size(0)
    C = torch.empty((M, N), dtype=out_dtype, device=xq.device)
    p = capi.GgufMmvqParams(M=M, N=int(N), K=int(K), A=None, B=B_packed.data_ptr(),
                            C=C.data_ptr(), type=int(type),
                            out_dtype=capi.DTYPE_F32 if out_dtype == torch.float32 else capi.DTYPE_BF16)
    capi.check(_lib.lsg_gguf_mmvq_q8_1(ctypes.byref(p), _ptr(xq), _stream()))
    return C


def gguf_dequant_gemm(A, B_packed, type, N, K, out_dtype=torch.bfloat16):
    """Lossless-activation golden: bf16 A @ dequant(B)^T (fp32 accumulate).

    Mirrors launch_gguf_dequant_gemm (csrc/sm120/gemm/gguf/gguf_dequant_gemm.cu:309-325),
    which the reference reaches from Python through gguf_grouped_gemm(strategy=0).
    """
    _require(A.is_cuda and A.dtype == torch.bfloat16 and A.is_contiguous(),
             "gguf_dequant_gemm: A must be contiguous BF16 on CUDA")
    M = A.size(0)
    C = torch.empty((M, N), dtype=out_dtype, device=A.device)
    p = _gemm_params(A, B_packed, C, type, N, K,
                     capi.DTYPE_F32 if out_dtype == torch.float32 else capi.DTYPE_BF16)
    capi.check(_lib.lsg_gguf_dequant_gemm(ctypes.byref(p), _stream()))
    return C


def gguf_dequant(B_packed, type):
    """Packed blocks uint8 [N, row_bytes] -> fp32 [N, K]."""
    t = int(type)
    N = B_packed.size(0)
    nblk = B_packed.size(1) // capi.BLOCK_BYTES[t]
    out = torch.empty((N, nblk * capi.BLOCK_VALUES[t]), dtype=torch.float32, device=B_packed.device)
    capi.check(_lib.lsg_gguf_dequant_blocks(_ptr(B_packed), _ptr(out), t, N * nblk, _stream()))
    return out
