"""Single-shape probe of the GGUF mat-vec, for profilers and quick timing.

    python -m layerstormgemmkernels_b200.probe TYPE N K M COPIES CALLS [--time] [--mmq]

Makes COPIES device copies of one random-byte weight of the given type and shape (so that
successive calls stream from DRAM, not from L2), quantizes an M x K activation once, and
issues CALLS mat-vec calls through the C ABI, walking over the copies.  With --time it
also reports CUDA-event time per call from a CUDA-graph replay.  With --mmq the calls go to
the tensor-core GEMM (lsg_gguf_mmq) instead of the mat-vec.
"""
import sys

import torch

from . import capi, ops, quantize as Q


def main(argv):
    name, N, K, M, copies, calls = argv[0], *map(int, argv[1:6])
    t = capi.GGUF_TYPES[name]
    base = torch.from_numpy(Q.random_gguf_weight(name, N, K, seed=1)).cuda()
    weights = [base.clone() for _ in range(copies)]
    A = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    xq = ops.quantize_q8_1(A)
    if "--mmq" in argv:
        def call(w):
            return ops.gguf_mmq(A, w, t, N, K)
    else:
        def call(w):
            return ops.gguf_mmvq_q8_1(xq, w, t, N, K)
    for i in range(calls):
        call(weights[i % copies])
    torch.cuda.synchronize()
    if "--time" in argv:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for w in weights:
                call(w)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (20 * copies)
        nbytes = N * (K // capi.BLOCK_VALUES[t]) * capi.BLOCK_BYTES[t] + M * K * 2 + M * N * 2
        print(f"{name} N={N} K={K} M={M}: {us:.2f} us per call, {nbytes / us / 1e3:.0f} GB/s, "
              f"{2.0 * M * N * K / us / 1e6:.1f} TFLOP/s")
    print("device status", capi.device_status())


if __name__ == "__main__":
    main(sys.argv[1:])
