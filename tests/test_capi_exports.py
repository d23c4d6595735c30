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


def test_batch_workspace_plans_need_no_gpu(built_lib):
    """The workspace of the batched mat-vec entries is planned on the host: the device batch
    needs the largest Q8_1 image, the host-memory batch one staged copy and one image per
    distinct activation plus result rows per projection; argument errors come back before
    any CUDA call."""
    from layerstormgemmkernels_b200 import capi
    import pytest

    def a256(v):
        return (v + 255) & ~255

    P = capi.GgufMmvqParams
    # pointers are only compared, never dereferenced, by the planning functions
    shapes = [(4096, 4096, 0x1000), (1024, 4096, 0x1000), (1024, 4096, 0x1000),
              (4096, 4096, 0x2000), (14336, 4096, 0x3000), (14336, 4096, 0x3000), (4096, 14336, 0x4000)]
    arr = (P * len(shapes))()
    for i, (N, K, A) in enumerate(shapes):
        arr[i] = P(M=2, N=N, K=K, A=A, B=0x10, C=0x20 + i, type=capi.Q4_K, out_dtype=0)
    assert capi.lib.lsg_gguf_mmvq_batch_workspace_bytes(arr, len(shapes)) == 2 * (14336 // 32) * 36
    want = sum(a256(2 * N * 4) for N, _, _ in shapes)
    for K in (4096, 4096, 4096, 14336):           # four distinct activations
        want += a256(2 * K * 2) + a256(2 * (K // 32) * 36)
    assert capi.lib.lsg_gguf_mmvq_host_batch_workspace_bytes(arr, len(shapes)) == want
    assert capi.lib.lsg_gguf_mmvq_host_workspace_bytes(2, 4096, 4096) == \
        a256(2 * 4096 * 2) + a256(2 * 128 * 36) + a256(2 * 4096 * 4)
    assert capi.lib.lsg_gguf_mmvq_host_batch_workspace_bytes(arr, 65) == 0   # more than 64 entries

    bad = (P * 2)()
    bad[0] = arr[0]
    bad[1] = P(M=1, N=8, K=100, A=0x1000, B=0x10, C=0x20, type=capi.Q4_K, out_dtype=0)
    for fn in (capi.lib.lsg_gguf_mmvq_batch, capi.lib.lsg_gguf_mmvq_host_batch):
        with pytest.raises(ValueError, match="divisible by 256"):
            capi.check(fn(bad, 2, None, 0, None))
        with pytest.raises(capi.LsgError):
            capi.check(fn(arr, len(shapes), None, 0, None))     # no workspace
        assert fn(arr, 0, None, 0, None) == 0                     # empty batch
