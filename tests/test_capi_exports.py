"""CPU test: the C-ABI library builds, loads, and exports every symbol include/lsg.h declares."""
import ctypes
import os
import re


def test_library_exports_every_declared_symbol(built_lib):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, "include", "lsg.h")) as f:
        header = f.read()
    declared = sorted(set(re.findall(r"LSG_API\s+[\w\s\*]+?\b(lsg_\w+)\s*\(", header)))
    assert len(declared) >= 10
    lib = ctypes.CDLL(built_lib)
    missing = [n for n in declared if not hasattr(lib, n)]
    assert not missing, f"declared in lsg.h but not exported: {missing}"
    from layerstormgemmkernels_b200 import capi
    assert set(capi.EXPORTS) == set(declared), set(capi.EXPORTS) ^ set(declared)


def test_argument_errors_need_no_gpu(built_lib):
    """Validation happens on the host before any CUDA call."""
    from layerstormgemmkernels_b200 import capi
    import pytest
    p = capi.GgufMmvqParams(M=1, N=8, K=100, A=None, B=None, C=None, type=capi.Q4_K, out_dtype=0)
    with pytest.raises(ValueError, match="divisible by 256"):
        capi.check(capi.lib.lsg_gguf_mmvq(ctypes.byref(p), None, 0, None))
    p = capi.GgufMmvqParams(M=1, N=8, K=256, A=None, B=None, C=None, type=42, out_dtype=0)
    with pytest.raises(capi.LsgError):
        capi.check(capi.lib.lsg_gguf_mmvq(ctypes.byref(p), None, 0, None))
    assert capi.lib.lsg_gguf_mmvq_workspace_bytes(3, 4096) == 3 * 128 * 36
    assert capi.lib.lsg_gguf_block_bytes(capi.Q6_K) == 210
    assert capi.lib.lsg_gguf_block_values(capi.Q4_0) == 32
