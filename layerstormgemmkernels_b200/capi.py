"""ctypes view of the C ABI declared in include/lsg.h.

The shared library is the product; this module only loads it and turns status
codes into exceptions.  There is no CPU fallback: if liblsg_b200.so is missing
or does not load, importing this module raises.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liblsg_b200.so")

from .formats import (Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, Q8_0, MXFP4, Q4_0, GGUF_TYPES, BLOCK_BYTES,  # noqa: F401
                      BLOCK_VALUES, DTYPE_BF16, DTYPE_F32, DTYPE_F16)

LSG_OK = 0
LSG_ERR_INVALID = -1
LSG_ERR_UNSUPPORTED = -2
LSG_ERR_WORKSPACE = -3
LSG_ERR_CUDA = -4
LSG_ERR_ALIGNMENT = -5
LSG_ERR_DEVICE_WAIT = -6


class LsgError(RuntimeError):
    """A C-ABI call returned a negative status.  `.code` holds it."""

    def __init__(self, code, message):
        super().__init__(f"lsg status {code}: {message}")
        self.code = code


class LsgInvalidArgument(LsgError, ValueError):
    """LSG_ERR_INVALID: where the reference's launchers throw std::invalid_argument."""


class GgufMmvqParams(ctypes.Structure):
    _fields_ = [("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
                ("A", ctypes.c_void_p), ("B", ctypes.c_void_p), ("C", ctypes.c_void_p),
                ("type", ctypes.c_int), ("out_dtype", ctypes.c_int)]


class DynamicFp8QuantParams(ctypes.Structure):
    _fields_ = [("num_tokens", ctypes.c_int), ("hidden_size", ctypes.c_int),
                ("input", ctypes.c_void_p), ("output", ctypes.c_void_p),
                ("scales", ctypes.c_void_p), ("m_major_scales", ctypes.c_int)]


class Nvfp4GroupedQuantParams(ctypes.Structure):
    _fields_ = [("input", ctypes.c_void_p), ("up", ctypes.c_void_p),
                ("output_packed", ctypes.c_void_p), ("output_scales", ctypes.c_void_p),
                ("expert_offsets", ctypes.c_void_p), ("sf_offsets", ctypes.c_void_p),
                ("total_tokens", ctypes.c_int), ("num_experts", ctypes.c_int),
                ("K", ctypes.c_int), ("input_scales", ctypes.c_void_p)]


class GgufGroupedGemmParams(ctypes.Structure):
    _fields_ = [("type", ctypes.c_int), ("strategy", ctypes.c_int), ("num_experts", ctypes.c_int),
                ("N", ctypes.c_int), ("K", ctypes.c_int), ("A_base", ctypes.c_void_p),
                ("D_base", ctypes.c_void_p), ("expert_offsets", ctypes.c_void_p),
                ("B_ptrs", ctypes.c_void_p), ("out_dtype", ctypes.c_int)]


class GgufMoeFfnParams(ctypes.Structure):
    _fields_ = [("type", ctypes.c_int), ("num_experts", ctypes.c_int), ("H", ctypes.c_int), ("I", ctypes.c_int),
                ("A_base", ctypes.c_void_p), ("D_base", ctypes.c_void_p), ("expert_offsets", ctypes.c_void_p),
                ("gate_ptrs", ctypes.c_void_p), ("up_ptrs", ctypes.c_void_p), ("down_ptrs", ctypes.c_void_p),
                ("out_dtype", ctypes.c_int), ("perm", ctypes.c_void_p), ("top_k", ctypes.c_int)]


class Fp8GemmParams(ctypes.Structure):
    _fields_ = [("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int), ("A", ctypes.c_void_p),
                ("B", ctypes.c_void_p), ("D", ctypes.c_void_p), ("scale_A", ctypes.c_void_p),
                ("scale_B", ctypes.c_void_p), ("output_dtype", ctypes.c_int)]


class Fp8GroupedGemmParams(ctypes.Structure):
    _fields_ = [("num_experts", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
                ("A_base", ctypes.c_void_p), ("B_base", ctypes.c_void_p), ("D_base", ctypes.c_void_p),
                ("scale_A_base", ctypes.c_void_p), ("scale_B_base", ctypes.c_void_p),
                ("expert_offsets", ctypes.c_void_p), ("problem_sizes", ctypes.c_void_p),
                ("output_dtype", ctypes.c_int), ("B_ptrs", ctypes.c_void_p), ("scale_B_ptrs", ctypes.c_void_p)]


class Nvfp4GemmParams(ctypes.Structure):
    _fields_ = [("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int), ("A", ctypes.c_void_p),
                ("B", ctypes.c_void_p), ("D", ctypes.c_void_p), ("scale_A", ctypes.c_void_p),
                ("scale_B", ctypes.c_void_p), ("alpha", ctypes.c_float), ("output_dtype", ctypes.c_int)]


class Nvfp4GroupedGemmParams(ctypes.Structure):
    _fields_ = [("num_experts", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
                ("A_base", ctypes.c_void_p), ("B_base", ctypes.c_void_p), ("D_base", ctypes.c_void_p),
                ("scale_A_base", ctypes.c_void_p), ("scale_B_base", ctypes.c_void_p),
                ("alphas", ctypes.c_void_p), ("expert_offsets", ctypes.c_void_p),
                ("sf_offsets", ctypes.c_void_p), ("problem_sizes", ctypes.c_void_p),
                ("output_dtype", ctypes.c_int), ("B_ptrs", ctypes.c_void_p),
                ("scale_B_ptrs", ctypes.c_void_p)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m layerstormgemmkernels_b200.build` "
            "(there is no CPU fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    vp, ci, sz, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_longlong
    sigs = {
        "lsg_last_error": (ctypes.c_char_p, []),
        "lsg_version": (ctypes.c_char_p, []),
        "lsg_device_status": (ci, [ctypes.POINTER(ci)]),
        "lsg_set_wait_limit_cycles": (ci, [ll]),
        "lsg_test_mmvq_drop_slab": (ci, [ci]),
        "lsg_ep_barrier": (ci, [vp, ci, ci, ci, vp]),
        "lsg_gguf_block_values": (ci, [ci]),
        "lsg_gguf_block_bytes": (ci, [ci]),
        "lsg_quantize_q8_1": (ci, [vp, vp, ci, ci, vp]),
        "lsg_gguf_mmvq_workspace_bytes": (sz, [ci, ci]),
        "lsg_gguf_mmvq": (ci, [ctypes.POINTER(GgufMmvqParams), vp, sz, vp]),
        "lsg_gguf_mmvq_q8_1": (ci, [ctypes.POINTER(GgufMmvqParams), vp, vp]),
        "lsg_gguf_mmvq_batch_workspace_bytes": (sz, [ctypes.POINTER(GgufMmvqParams), ci]),
        "lsg_gguf_mmvq_batch": (ci, [ctypes.POINTER(GgufMmvqParams), ci, vp, sz, vp]),
        "lsg_gguf_mmvq_batch_plan": (ci, [ctypes.POINTER(GgufMmvqParams), ci, ctypes.POINTER(ci), ctypes.POINTER(ci),
                                          ctypes.POINTER(ci), ci]),
        "lsg_gguf_mmvq_host_workspace_bytes": (sz, [ci, ci, ci]),
        "lsg_gguf_mmvq_host": (ci, [ctypes.POINTER(GgufMmvqParams), vp, sz, vp]),
        "lsg_gguf_mmvq_host_batch_workspace_bytes": (sz, [ctypes.POINTER(GgufMmvqParams), ci]),
        "lsg_gguf_mmvq_host_batch": (ci, [ctypes.POINTER(GgufMmvqParams), ci, vp, sz, vp]),
        "lsg_gguf_mmvq_noalloc": (ci, [ctypes.POINTER(GgufMmvqParams), vp]),
        "lsg_mmvq_set_tuning": (ci, [ci, ci, ci, ci, ci]),
        "lsg_mmq_set_weight_path": (ci, [ci]),
        "lsg_gguf_mmq_gather": (ci, [ctypes.POINTER(GgufMmvqParams), vp, ci, ci, ci, vp, sz, vp]),
        "lsg_gguf_mmq_gather_mc": (ci, [ctypes.POINTER(GgufMmvqParams), vp, ci, ci, ci, vp, vp, sz, vp]),
        "lsg_gguf_gemm_bf16_workspace_bytes": (sz, [ci, ci, ci]),
        "lsg_gguf_gemm_bf16": (ci, [ctypes.POINTER(GgufMmvqParams), vp, sz, vp]),
        "lsg_dynamic_fp8_quant": (ci, [ctypes.POINTER(DynamicFp8QuantParams), vp]),
        "lsg_bf16_to_nvfp4_grouped": (ci, [ctypes.POINTER(Nvfp4GroupedQuantParams), vp]),
        "lsg_silu_mul_to_nvfp4_grouped": (ci, [ctypes.POINTER(Nvfp4GroupedQuantParams), vp]),
        "lsg_nvfp4_sf_offsets": (ci, [vp, vp, ci, vp]),
        "lsg_gguf_grouped_gemm_workspace_bytes": (sz, [ci, ci, ci]),
        "lsg_gguf_grouped_gemm": (ci, [ctypes.POINTER(GgufGroupedGemmParams), ci, vp, sz, ci, vp]),
        "lsg_fp8_gemm_workspace_bytes": (sz, [ci, ci, ci]),
        "lsg_fp8_gemm": (ci, [ctypes.POINTER(Fp8GemmParams), vp, sz, vp]),
        "lsg_fp8_grouped_gemm_workspace_bytes": (sz, [ci, ci, ci, ci]),
        "lsg_fp8_grouped_gemm": (ci, [ctypes.POINTER(Fp8GroupedGemmParams), ci, vp, sz, vp]),
        "lsg_weight_fp8_quant": (ci, [vp, vp, vp, ci, ci, vp]),
        "lsg_bf16_to_nvfp4": (ci, [vp, vp, vp, ci, ci, vp]),
        "lsg_nvfp4_dequant_bf16": (ci, [vp, vp, ctypes.c_float, vp, ci, ci, vp]),
        "lsg_nvfp4_gemm_workspace_bytes": (sz, [ci, ci, ci]),
        "lsg_nvfp4_gemm": (ci, [ctypes.POINTER(Nvfp4GemmParams), vp, sz, vp]),
        "lsg_gguf_moe_ffn_workspace_bytes": (sz, [ci, ci, ci, ci]),
        "lsg_gguf_moe_ffn": (ci, [ctypes.POINTER(GgufMoeFfnParams), ci, vp, sz, vp]),
        "lsg_gguf_moe_ffn_set_matvec_rows": (ci, [ci]),
        "lsg_build_active_expert_list": (ci, [vp, ci, ci, vp, vp]),
        "lsg_build_mmq_tile_map": (ci, [vp, ci, ci, ci, vp, vp, vp]),
        "lsg_gguf_grouped_gemm_workspace_bytes_ex": (sz, [ci, ci, ci, ci]),
        "lsg_gguf_mmq_workspace_bytes": (sz, [ci, ci, ci]),
        "lsg_gguf_mmq": (ci, [ctypes.POINTER(GgufMmvqParams), vp, sz, vp]),
        "lsg_nvfp4_grouped_gemm_workspace_bytes": (sz, [ci, ci, ci, ci]),
        "lsg_nvfp4_grouped_gemm_workspace_bytes_ex": (sz, [ci, ci, ci, ci, ci]),
        "lsg_nvfp4_grouped_gemm": (ci, [ctypes.POINTER(Nvfp4GroupedGemmParams), ci, vp, sz, vp]),
        "lsg_nvfp4_sf_buffer_bytes": (sz, [ci, ci]),
        "lsg_nvfp4_reformat_scales": (ci, [vp, vp, ci, ci, vp]),
        "lsg_moe_route": (ci, [vp, ci, ci, ci, vp, vp, vp]),
        "lsg_ep_expert_order": (ci, [vp, ci, ci, ci, vp, vp, vp, vp, vp]),
        "lsg_ep_publish_counts": (ci, [vp, ci, ci, ci, vp, vp]),
        "lsg_ep_plan": (ci, [vp, ci, ci, ci, ci, vp, vp, vp, vp, vp, vp]),
        "lsg_ep_send_rows": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, ci, vp, ci, vp, vp]),
        "lsg_ep_return_rows": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, vp, vp]),
        "lsg_ep_send_rows_group": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, ci, vp, ci, vp, ci, ci, vp]),
        "lsg_ep_return_rows_group": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, vp, vp, ci, ci, vp]),
        "lsg_moe_permutation_scratch_ints": (ctypes.c_longlong, [ci, ci, ci]),
        "lsg_moe_permutation": (ci, [vp, ci, ci, ci, vp, vp, vp, vp, vp]),
        "lsg_moe_permute": (ci, [vp, vp, ci, ci, ci, vp, vp]),
        "lsg_moe_unpermute": (ci, [vp, vp, vp, ci, ci, ci, vp, vp]),
        "lsg_gguf_dequant_gemm": (ci, [ctypes.POINTER(GgufMmvqParams), vp]),
        "lsg_gguf_dequant_blocks": (ci, [vp, vp, ci, ll, vp]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib, sorted(sigs)


lib, EXPORTS = _load()


def check(status):
    """Raises the exception matching a negative lsg_status."""
    if status == LSG_OK:
        return
    msg = lib.lsg_last_error().decode("utf-8", "replace")
    if status == LSG_ERR_INVALID:
        raise LsgInvalidArgument(status, msg)
    raise LsgError(status, msg)


def device_status():
    """Reads and clears the device-side status word (synchronizes the device)."""
    code = ctypes.c_int(0)
    check(lib.lsg_device_status(ctypes.byref(code)))
    return code.value
