"""How lsg_gguf_mmvq_batch splits a batch into launches and which launches may skip the wait for
the one in front of them (lsg_gguf_mmvq_batch_plan: host arithmetic on the parameter blocks, no
GPU).  The rule under test: entries of one shape share a launch when they read the same
activations or share no buffer at all; a launch is released from the wait only when it shares
no buffer with ANY earlier entry of the call."""
import ctypes
import os
import subprocess
import sys

import pytest

from layerstormgemmkernels_b200 import capi

P = capi.GgufMmvqParams
Q4_K = capi.GGUF_TYPES["Q4_K"]


def plan(entries, out_dtype=capi.DTYPE_BF16):
    arr = (P * max(len(entries), 1))(*[P(M=M, N=N, K=K, A=A, B=0x1000, C=C, type=Q4_K, out_dtype=out_dtype)
                                       for (M, N, K, A, C) in entries])
    f, c, k = (ctypes.c_int * 32)(), (ctypes.c_int * 32)(), (ctypes.c_int * 32)()
    n = capi.lib.lsg_gguf_mmvq_batch_plan(arr, len(entries), f, c, k, 32)
    return [(f[i], c[i], k[i]) for i in range(n)]


X, ATT, H, ACT = 0x100000, 0x200000, 0x300000, 0x400000    # activations, 1 MB apart
OUT = [0x1000000 + i * 0x100000 for i in range(16)]         # results, 1 MB apart


def layer(M=1):
    return [(M, 4096, 4096, X, OUT[0]), (M, 1024, 4096, X, OUT[1]), (M, 1024, 4096, X, OUT[2]),
            (M, 4096, 4096, ATT, OUT[3]), (M, 14336, 4096, H, OUT[4]), (M, 14336, 4096, H, OUT[5]),
            (M, 4096, 14336, ACT, OUT[6])]


def test_decoder_layer_is_two_launches_and_the_second_does_not_wait():
    assert plan(layer()) == [(0, 6, 1), (6, 1, 2)]


def test_batch_rows_above_the_in_kernel_quantizer_keep_waiting_launches():
    # 4 x 14336 values are above the limit: down gets a quantizer launch and waits; nothing
    # after the first launch can skip its wait, so the first launch is an ordinary one
    assert plan(layer(4)) == [(0, 6, 0), (6, 1, 4)]
    # 16 rows: nothing is quantized inside the mat-vec, so only entries with the same A join
    assert plan(layer(16)) == [(0, 3, 4), (3, 1, 4), (4, 2, 4), (6, 1, 4)]


def test_chained_entries_stay_in_order():
    y0, y1 = OUT[0], OUT[1]
    assert plan([(1, 4096, 4096, X, y0), (1, 1024, 4096, y0, y1)]) == [(0, 1, 0), (1, 1, 0)]


def test_mixed_batch():
    y0, y1, y2, y3, y4 = OUT[:5]
    x2, x3 = 0x500000, 0x600000
    entries = [
        (1, 4096, 4096, X, y0),      # 0
        (1, 1024, 4096, x2, y2),     # 1: own input, shares nothing with 0 -> same launch
        (1, 2048, 4096, y0, y1),     # 2: reads the result of 0 -> its own launch, waits
        (1, 1024, 2048, x3, y3),     # 3: independent of everything before it -> does not wait
        (1, 1024, 2048, y1, y4),     # 4: same shape as 3 but reads the result of 2 -> waits
        (1, 1024, 4096, X, y2),      # 5: rewrites the result of 1 -> waits
    ]
    assert plan(entries) == [(0, 2, 1), (2, 1, 0), (3, 1, 2), (4, 1, 0), (5, 1, 0)]


def test_partial_overlap_of_results_counts_as_shared():
    # entry 1's result starts inside entry 0's result (4096 bf16 = 8192 bytes)
    assert plan([(1, 4096, 4096, X, OUT[0]), (1, 4096, 4096, ATT, OUT[0] + 8190)]) == [(0, 1, 0), (1, 1, 0)]
    assert plan([(1, 4096, 4096, X, OUT[0]), (1, 4096, 4096, ATT, OUT[0] + 8192)]) == [(0, 2, 0)]
    # an entry that writes what an earlier one reads
    assert plan([(1, 4096, 4096, X, OUT[0]), (1, 2048, 2048, ATT, X + 4096)]) == [(0, 1, 0), (1, 1, 0)]
    # float results are twice as long
    assert plan([(1, 4096, 4096, X, OUT[0]), (1, 4096, 4096, ATT, OUT[0] + 8192)],
                out_dtype=capi.DTYPE_F32) == [(0, 1, 0), (1, 1, 0)]


def test_empty_entries_and_long_runs():
    assert plan([]) == []
    assert plan([(0, 4096, 4096, X, OUT[0]), (1, 0, 4096, X, OUT[1])]) == []
    # an empty entry in front does not make the next one "not the first launch"
    assert plan([(0, 16, 4096, X, OUT[9])] + layer()) == [(1, 6, 1), (7, 1, 2)]
    # eight projections of one input: six per launch; the second launch shares no result with
    # the first and does not wait
    eight = [(1, 256, 4096, X, OUT[i]) for i in range(8)]
    assert plan(eight) == [(0, 6, 1), (6, 2, 2)]


def test_environment_switch_restores_waiting_launches():
    code = ("import tests.test_batch_plan as t; "
            "assert t.plan(t.layer()) == [(0, 3, 0), (3, 1, 0), (4, 2, 0), (6, 1, 0)], t.plan(t.layer())")
    env = dict(os.environ, LSG_MMVQ_BATCH_OVERLAP="0")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr


def test_null_params_are_rejected():
    assert capi.lib.lsg_gguf_mmvq_batch_plan(None, 3, None, None, None, 0) < 0


def test_bench_counts_its_launches_with_the_planner():
    """bench.py reports gpu_launches from the library's own plan of its layer."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    import bench
    def arr_of(entries):
        return (P * len(entries))(*[P(M=M, N=N, K=K, A=A, B=0x1000, C=C, type=Q4_K, out_dtype=capi.DTYPE_BF16)
                                    for (M, N, K, A, C) in entries])
    assert bench.planned_launches(capi, arr_of(layer(1)), 7) == (2, 2)
    assert bench.planned_launches(capi, arr_of(layer(8)), 7) == (2, 3)      # down: quantizer + mat-vec
    assert bench.planned_launches(capi, arr_of(layer(16)), 7) == (4, 8)
