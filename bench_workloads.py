"""The workloads of bench.py besides the headline decode layer: the MoE layer (expert-parallel
over the ranks), the prefill GEMM (column-split over the ranks), the NVFP4 expert block, the
activation quantizers, and a single-shape mode for profilers.  Each function returns one
result line (a dict in bench.py's JSON format); bench.py prints them.

Every function takes `ctx`: rank, world, dev (torch device), and times with CUDA events on
the current stream, max over ranks.  Nothing here touches the CPU oracle except the
`cpu_*` functions at the end, which are the bounded CPU baselines that sit beside the GPU
numbers (rank 0, one GPU).
"""
import ctypes
import json
import os
import sys
import time
from types import SimpleNamespace

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return SimpleNamespace(hbm=float(p["hbm_gbs"]), tf_burst=float(p["bf16_tflops"]),
                               tf=float(p["bf16_tflops_sustained"]), kind="measured")
    return SimpleNamespace(hbm=6650.0, tf_burst=1590.0, tf=1400.0, kind="fallback")


def time_steps(step, steps, warmup, ctx, flush=None):
    """CUDA-event time per step in ms, max over ranks; barrier + synchronize on both sides."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if ctx.world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if ctx.world > 1:
        t = torch.tensor([ms], device=ctx.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps


def _q4k(t):
    from layerstormgemmkernels_b200 import quantize as Q
    return Q.quantize_q4_k(t.numpy())


# --------------------------------------------------------------------------------------
# MoE layer: 128 experts, top-8, hidden 2048, expert FFN 768, Q4_K
# --------------------------------------------------------------------------------------
MOE = dict(E=128, k=8, H=2048, I=768)


def moe_expert_weights(dev, e0, e1, distinct=8):
    """Packed Q4_K gate / up / down matrices of experts e0..e1-1: `distinct` different experts
    quantized from N(0, 0.02) seed 3, tiled over the expert ids (every expert still has its own
    copy in HBM, so the weight traffic is that of 128 different experts)."""
    H, I = MOE["H"], MOE["I"]
    g = torch.Generator().manual_seed(3)
    base = []
    for _ in range(distinct):
        base.append((_q4k(torch.randn(I, H, generator=g) * 0.02), _q4k(torch.randn(I, H, generator=g) * 0.02),
                     _q4k(torch.randn(H, I, generator=g) * 0.02)))
    sets = [[torch.from_numpy(base[e % distinct][j]).to(dev) for e in range(e0, e1)] for j in range(3)]
    ptrs = [torch.tensor([w.data_ptr() for w in ws], dtype=torch.int64, device=dev) for ws in sets]
    return base, sets, ptrs


def run_moe(ctx, tokens, steps, warmup, weak=False, ep="peer", check=True, chunks=1, groups=1):
    from layerstormgemmkernels_b200 import capi, ops, distributed as D
    E, k, H, I = MOE["E"], MOE["k"], MOE["H"], MOE["I"]
    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    T_total = tokens * world if weak else tokens
    if T_total % world != 0:
        raise SystemExit("tokens must be divisible by the number of GPUs")
    T = T_total // world
    t = capi.Q4_K
    e0, e1 = D.expert_range(rank, world, E)
    _base, _sets, (gate_p, up_p, down_p) = moe_expert_weights(dev, e0, e1)
    gg = torch.Generator().manual_seed(1000 + rank)
    hidden = torch.randn(T, H, generator=gg).to(torch.bfloat16).to(dev)
    logits = torch.randn(T, E, generator=gg).to(dev)
    hidden_host, logits_host = hidden.cpu().pin_memory(), logits.cpu().pin_memory()

    def ffn(rows, offs, lo=None, hi=None):
        if lo is None:
            return ops.gguf_moe_ffn(rows, offs, gate_p, up_p, down_p, t, H, I)
        # one group of this rank's experts (EpPeerGroups): slices of the pointer arrays
        return ops.gguf_moe_ffn(rows, offs, gate_p[lo:hi], up_p[lo:hi], down_p[lo:hi], t, H, I)

    exchange, ep_mode = None, "single"
    if world > 1:
        ep_mode = ep
        if ep == "peer":
            try:
                # chunks > 1: halves of the tokens on side streams, one half's row exchange under the
                # other half's expert GEMMs.  Measured slower on this layer (each half repeats the
                # decoding of every expert's weights), so one exchange is the default.
                if chunks > 1 and T % chunks == 0 and T // chunks >= 64:
                    exchange = D.EpPeerPipeline.make(E, k, H, T, chunks=chunks)
                elif groups > 1 and (e1 - e0) >= groups and T * k // E > 8:
                    # groups of local experts on side streams: one group's rows travel while the
                    # other group's expert GEMMs run.  Also measured slower here (two GPUs, weak:
                    # 0.870 ms in two groups, 1.059 in four, 0.787 plain): every group is four more
                    # launches of persistent kernels over half as many items
                    exchange = D.EpPeerGroups.make(E, k, H, T, groups=groups)
                else:
                    exchange = D.EpPeerExchange.make(E, k, H, T)
            except Exception as exc:   # noqa: BLE001 - the optional path falls back
                if rank == 0:
                    print(f"peer-memory exchange unavailable ({type(exc).__name__}: {exc}); using NCCL all-to-all",
                          file=sys.stderr)
                ep_mode = "nccl"

    def layer(h, lg):
        if world == 1:
            idx, w = ops.moe_route(lg, k)
            offs, perm, inv = ops.moe_permutation(idx, E)
            # the permute (gather) is folded into the expert block's first operand preparation
            y = ops.gguf_moe_ffn(h, offs, gate_p, up_p, down_p, t, H, I, perm=perm, top_k=k)
            return ops.moe_unpermute(y, inv, w)
        if exchange is not None:
            return exchange.layer(h, lg, ffn, ops.moe_route, ops.moe_permutation, ops.moe_unpermute)
        return D.ep_moe_layer(h, lg, k, E, ffn, ops.moe_route, ops.moe_permutation, ops.moe_permute,
                              ops.moe_unpermute)

    equal = None
    if world > 1 and check and exchange is not None:
        # the scaling run proves itself: the peer-memory layer against the NCCL all-to-all layer
        a = layer(hidden, logits).clone()
        b = D.ep_moe_layer(hidden, logits, k, E, ffn, ops.moe_route, ops.moe_permutation, ops.moe_permute,
                           ops.moe_unpermute)
        ok = torch.tensor([1 if torch.equal(a, b) else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        equal = bool(ok.item())
    # The layer as a serving stack runs it: captured once into a CUDA graph and replayed (every
    # kernel of it is stream-ordered, nothing reads back to the host, and the cross-GPU barrier
    # keeps its count on the device).  The NCCL fallback exchange copies split sizes to the
    # host and stays eager.
    graphed = world == 1 or exchange is not None
    if graphed:
        for _ in range(2):
            layer(hidden, logits)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            graph_out = layer(hidden, logits)
        ms = time_steps(graph.replay, steps, warmup, ctx)
        del graph_out
    else:
        ms = time_steps(lambda: layer(hidden, logits), steps, warmup, ctx)
    overflow = bool(exchange is not None and exchange.overflowed())
    gemm_ms = None
    if world == 1:
        idx, _w = ops.moe_route(logits, k)
        offs, perm, _inv = ops.moe_permutation(idx, E)
        rows = ops.moe_permute(hidden, perm, k)
        gemm_ms = time_steps(lambda: ffn(rows, offs), steps, warmup, ctx)

    def e2e_step():
        h = hidden_host.to(dev, non_blocking=True)
        lg = logits_host.to(dev, non_blocking=True)
        return layer(h, lg).cpu()
    e2e_ms = time_steps(e2e_step, max(3, min(steps, 20)), 3, ctx)

    flops = 6.0 * T_total * k * H * I
    pk = peaks()
    value = flops / (ms * 1e-3) / 1e12
    # T=1 and T=64 stream expert weights (21 MB / up to 340 MB): HBM-bound cells
    active = min(E, T_total * k)
    wbytes = active * 3 * (I * (H // 256) * 144)
    hbm_bound = T_total * k // E <= 8
    line = {
        "metric": "moe_grouped_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak" if weak else "strong", "vs_baseline": None, "dtype": "f16 (tcgen05, fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": f"MoE layer, 128 experts top-8, H=2048, I=768, Q4_K, {T_total} tokens: "
                               "route, permute, gate/up/down grouped GEMMs, SwiGLU, combine",
                   "tokens": T_total, "tokens_per_gpu": T,
                   "launch": "one CUDA graph per layer" if graphed else "eager (the NCCL exchange reads split sizes on the host)",
                   "parallelism": (f"ep{world}, rows exchanged by peer-memory stores"
                                   + (f" in {exchange.chunks} pipelined "
                                      + ("expert groups" if isinstance(exchange, D.EpPeerGroups) else "token chunks")
                                      if hasattr(exchange, "chunks") else "")
                                   + ", library flag barrier"
                                   if ep_mode == "peer" and exchange is not None
                                   else f"ep{world}, NCCL all-to-all" if world > 1 else "single"),
                   "l2_defeat": "339 MB of expert weights (per rank set) exceed the 126 MB L2"},
        "roofline": ({"bound": "hbm", "achieved": wbytes / (ms * 1e-3) / 1e9 / world, "peak": pk.hbm, "unit": "GB/s",
                      "frac": wbytes / (ms * 1e-3) / 1e9 / world / pk.hbm, "peak_kind": pk.kind, "traffic": None,
                      "note": f"decode-sized batch: weight bytes of the {active} routed experts over the layer time"}
                     if hbm_bound else
                     {"bound": "tensor", "achieved": value / world, "peak": pk.tf, "unit": "TFLOP/s",
                      "frac": value / world / pk.tf, "peak_kind": f"{pk.kind} (cuBLAS bf16, sustained)",
                      "traffic": None,
                      "note": "whole layer (routing, permute, expert block, combine) over the GEMM flops"}),
        "expert_block": None if gemm_ms is None else {
            "what": "lsg_gguf_moe_ffn alone on the routed rows: operand preparation, gate|up GEMM, SwiGLU, down GEMM",
            "ms": gemm_ms, "tflops": flops / (gemm_ms * 1e-3) / 1e12,
            "frac_of_peak": flops / (gemm_ms * 1e-3) / 1e12 / pk.tf},
        "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": T * H * 2 + T * E * 4, "d2h_bytes_per_step": T * H * 2},
        "gpu_launches": steps * (10 if world == 1 else 11),
    }
    if equal is not None:
        line["equal_to_nccl_exchange"] = equal
    if overflow:
        line["overflow"] = True
    return line


# --------------------------------------------------------------------------------------
# Prefill GEMM: Q4_K 14336 x 4096, M tokens, column split over the ranks
# --------------------------------------------------------------------------------------
def prefill_weight():
    g = torch.Generator().manual_seed(2)
    return (torch.randn(14336, 4096, generator=g) * 0.02)


def run_prefill(ctx, M, steps, warmup, ep="peer", w_full=None, check=True):
    from layerstormgemmkernels_b200 import capi, ops, distributed as D
    N, K = 14336, 4096
    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    t = capi.Q4_K
    n0, n1 = D.column_slab(rank, world, N)
    w = prefill_weight() if w_full is None else w_full
    slab = torch.from_numpy(_q4k(w[n0:n1])).to(dev)
    A = torch.randn(M, K, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(dev)
    A_host = A.cpu().pin_memory()
    fused_gather = None
    if world > 1 and ep == "peer":
        try:
            fused_gather = D.ColumnSplitPeer(M, N)
        except Exception as exc:   # noqa: BLE001
            if rank == 0:
                print(f"peer-memory gather unavailable ({type(exc).__name__}: {exc}); using NCCL all-gather",
                      file=sys.stderr)

    def step(a=A):
        if fused_gather is not None:
            return fused_gather.gemm(a, slab, t, K)
        out = ops.gguf_mmq(a, slab, t, n1 - n0, K)
        return out if world == 1 else D.column_split_gather(out)

    equal = None
    if world > 1 and check and fused_gather is not None:
        a = step().clone()
        # the same GEMM route with one local output (above 2048 rows the gather entry keeps the
        # prepared-operand kernel, whose results differ from the fused kernel's by fp16 rounding
        # of the weights), then NCCL's all-gather
        local = torch.empty((M, n1 - n0), dtype=torch.bfloat16, device=dev)
        ops.gguf_mmq_gather(A, slab, t, n1 - n0, K, torch.tensor([local.data_ptr()], dtype=torch.int64, device=dev),
                            n1 - n0, 0)
        b = D.column_split_gather(local)
        ok = torch.tensor([1 if torch.equal(a, b) else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        equal = bool(ok.item())
    ms = time_steps(step, steps, warmup, ctx)
    e2e_ms = time_steps(lambda: step(A_host.to(dev, non_blocking=True)).cpu(), max(3, min(steps, 10)), 3, ctx)
    flops = 2.0 * M * N * K
    pk = peaks()
    value = flops / (ms * 1e-3) / 1e12
    line = {
        "metric": "q4_k_mmq_prefill_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16 (tcgen05, fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": f"Q4_K 14336x4096 prefill GEMM, M={M}, Q8_1 activations",
                   "parallelism": ("single" if world == 1 else
                                   f"column-split x{world}, all-gather fused into the GEMM epilogue ("
                                   + ("multimem stores into the NVLink multicast object" if getattr(fused_gather, "multicast_ptr", 0)
                                      else "peer stores") + ")"
                                   if fused_gather is not None else f"column-split x{world} + NCCL all-gather"),
                   "l2_defeat": "weights 33 MB + activations + outputs (117 MB at M=4096) exceed L2 at M=4096; "
                                "at M=512 the operands fit L2 and the number is an L2-resident one"},
        "roofline": {"bound": "tensor", "achieved": value / world, "peak": pk.tf, "unit": "TFLOP/s",
                     "frac": value / world / pk.tf, "peak_kind": f"{pk.kind} (cuBLAS bf16, sustained)",
                     "traffic": None},
        "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2},
        "gpu_launches": steps * (3 if (M > 2048 and fused_gather is not None) else 2),
    }
    if equal is not None:
        line["equal_to_nccl_gather"] = equal
    return line


# --------------------------------------------------------------------------------------
# NVFP4 expert block: 8 experts, top-2, hidden 4096, FFN 14336, 4096 tokens
# --------------------------------------------------------------------------------------
NVFP4 = dict(E=8, k=2, H=4096, I=14336)


def nvfp4_expert_weights(dev, e0, e1, seed=4):
    """NVFP4 weights of experts e0..e1-1, quantized ON THE DEVICE by the library's own quantizer
    (lsg_bf16_to_nvfp4, bit-exact against the oracle in the tests) from bf16 N(0, 0.02)
    weights generated on the device with a seeded generator: the host packer would need
    minutes for 1.4 G values."""
    from layerstormgemmkernels_b200 import ops
    H, I = NVFP4["H"], NVFP4["I"]
    g = torch.Generator(device=dev).manual_seed(seed)
    out = []
    for shape in ((I, H), (I, H), (H, I)):
        codes, scales, alphas = [], [], []
        for _e in range(e0, e1):
            w = (torch.randn(shape, generator=g, device=dev) * 0.02).to(torch.bfloat16)
            s2 = float(w.float().abs().max().item()) / 6.0 / 448.0 * 448.0   # per-tensor scale: amax / 6
            s2 = max(s2, 1e-12)
            c, sf = ops.bf16_to_nvfp4((w.float() / s2).to(torch.bfloat16))
            codes.append(c)
            scales.append(sf)
            alphas.append(s2)
        out.append((torch.stack(codes), torch.stack(scales), torch.tensor(alphas, dtype=torch.float32, device=dev)))
    return out


def run_nvfp4(ctx, tokens, steps, warmup):
    """gate, up, SwiGLU + quantize, down over rows grouped by expert (top-2 of 8 experts, even
    routing), each projection one nvfp4_grouped_gemm call as in the reference's pairing test
    (tests/test_kernels.py:543-592)."""
    from layerstormgemmkernels_b200 import ops
    E, k, H, I = NVFP4["E"], NVFP4["k"], NVFP4["H"], NVFP4["I"]
    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    if E % world != 0:
        raise SystemExit("the NVFP4 block shards 8 experts: 1, 2, 4 or 8 GPUs")
    per = E // world
    rows = tokens * k // world                 # even routing: every rank's experts get their share
    (gc, gs, ga), (uc, us, ua), (dc, ds, da) = nvfp4_expert_weights(dev, rank * per, (rank + 1) * per)
    offs = torch.arange(per + 1, dtype=torch.int32, device=dev) * (rows // per)
    x = torch.randn(rows, H, generator=torch.Generator().manual_seed(7 + rank)).to(torch.bfloat16).to(dev)
    sizes_g = torch.tensor([[rows // per, I, H]] * per, dtype=torch.int32, device=dev)
    sizes_d = torch.tensor([[rows // per, H, I]] * per, dtype=torch.int32, device=dev)
    Dg = torch.empty((rows, I), dtype=torch.bfloat16, device=dev)
    Du = torch.empty((rows, I), dtype=torch.bfloat16, device=dev)
    Dd = torch.empty((rows, H), dtype=torch.bfloat16, device=dev)

    def step():
        xa, xs, sfo = ops.bf16_to_nvfp4_grouped(x, offs)
        ops.nvfp4_grouped_gemm(xa, gc, Dg, xs, gs, ga, offs, sfo, sizes_g, I, H, "bf16")
        ops.nvfp4_grouped_gemm(xa, uc, Du, xs, us, ua, offs, sfo, sizes_g, I, H, "bf16")
        aa, asf, sfo2 = ops.silu_mul_to_nvfp4_grouped(Dg, Du, offs)
        ops.nvfp4_grouped_gemm(aa, dc, Dd, asf, ds, da, offs, sfo2, sizes_d, H, I, "bf16")
        return Dd

    ms = time_steps(step, steps, warmup, ctx)
    flops = 6.0 * tokens * k * H * I
    pk = peaks()
    value = flops / (ms * 1e-3) / 1e12
    return {
        "metric": "nvfp4_grouped_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "e2m1 x e2m1, ue4m3 block scales (tcgen05 kind::mxf4nvf4, fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": f"NVFP4 expert block, 8 experts top-2, H=4096, I=14336, {tokens} tokens, even routing: "
                               "activation quantizer, gate, up, SwiGLU + quantizer, down",
                   "parallelism": "single" if world == 1 else f"ep{world} (experts sharded, rows local)",
                   "l2_defeat": "793 MB of packed expert weights exceed the 126 MB L2"},
        "roofline": {"bound": "tensor", "achieved": value / world, "peak": 4 * pk.tf, "unit": "TFLOP/s",
                     "frac": value / world / (4 * pk.tf),
                     "peak_kind": f"4 x the {pk.kind} cuBLAS bf16 sustained figure (no fp4 peak was measured)",
                     "traffic": None},
        "gpu_launches": steps * 8,
    }


# --------------------------------------------------------------------------------------
# Activation quantizers on a 4096 x 4096 bf16 tensor (HBM bound)
# --------------------------------------------------------------------------------------
def run_quant(ctx, steps, warmup):
    from layerstormgemmkernels_b200 import ops
    dev = ctx.dev
    M = K = 4096
    copies = 6                                       # 6 x 33.5 MB inputs > L2
    xs = [torch.randn(M, K, generator=torch.Generator().manual_seed(11 + i)).to(torch.bfloat16).to(dev)
          for i in range(copies)]
    offs = torch.tensor([0, M], dtype=torch.int32, device=dev)
    pk = peaks()
    cells = {}
    state = {"i": 0}

    def rot():
        state["i"] = (state["i"] + 1) % copies
        return xs[state["i"]]

    def cell(name, fn, bytes_per_call):
        # one CUDA graph over a call on each input copy: device time per call, without the host's
        # share of an eagerly issued 15 us kernel
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            keep = [fn() for _ in range(copies)]
        ms = time_steps(g.replay, max(2, steps // copies), max(1, warmup // copies), ctx) / copies
        del keep
        gbs = bytes_per_call / (ms * 1e-3) / 1e9
        cells[name] = {"ms": ms, "gbps": gbs, "frac_of_hbm_peak": gbs / pk.hbm, "bytes": bytes_per_call}

    cell("dynamic_fp8_quant", lambda: ops.dynamic_fp8_quant(rot()), M * K * 2 + M * K + M * (K // 128) * 4)
    cell("quantize_q8_1", lambda: ops.quantize_q8_1(rot()), M * K * 2 + M * (K // 32) * 36)
    # NVFP4 grouped: through the C ABI with caller-owned outputs.  The Python operator mirrors the
    # reference binding, which copies the offsets to the host on every call to size the scale buffer.
    from layerstormgemmkernels_b200 import capi
    packed = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
    scales = torch.zeros((M * (K // 16),), dtype=torch.uint8, device=dev)
    sf_offs = torch.tensor([0, M], dtype=torch.int32, device=dev)

    def nvfp4_call():
        x = rot()
        p = capi.Nvfp4GroupedQuantParams(input=x.data_ptr(), up=None, output_packed=packed.data_ptr(),
                                         output_scales=scales.data_ptr(), expert_offsets=offs.data_ptr(),
                                         sf_offsets=sf_offs.data_ptr(), total_tokens=M, num_experts=1, K=K,
                                         input_scales=None)
        capi.check(capi.lib.lsg_bf16_to_nvfp4_grouped(ctypes.byref(p), torch.cuda.current_stream().cuda_stream))
    cell("bf16_to_nvfp4_grouped", nvfp4_call, M * K * 2 + M * K // 2 + M * K // 16)
    best = cells["dynamic_fp8_quant"]
    return {
        "metric": "fp8_quant_gbps", "value": best["gbps"], "unit": "GB/s", "n_gpus": ctx.world, "steps": steps,
        "warmup": warmup, "ms_per_step": best["ms"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 -> e4m3 / int8 / e2m1", "data": "synthetic",
        "config": {"workload": "activation quantizers on a 4096x4096 bf16 tensor (dynamic FP8 headline; Q8_1 and "
                               "NVFP4 grouped in `cells`), each cell one CUDA graph over six calls (one per input copy)",
                   "l2_defeat": "calls rotate over six input tensors (201 MB)"},
        "roofline": {"bound": "hbm", "achieved": best["gbps"], "peak": pk.hbm, "unit": "GB/s",
                     "frac": best["gbps"] / pk.hbm, "peak_kind": pk.kind, "traffic": None},
        "cells": cells, "gpu_launches": steps * 3,
    }


# --------------------------------------------------------------------------------------
# One shape, a fixed number of calls: the command the profiler summaries are made with
# --------------------------------------------------------------------------------------
def run_shape(ctx, spec, calls, mmq=False, timed=True):
    """spec = "TYPE,N,K,M[,COPIES]".  Issues `calls` calls of the mat-vec (or, with mmq, the
    tensor-core GEMM) walking over COPIES device copies of one random-byte weight."""
    from layerstormgemmkernels_b200 import capi, ops, quantize as Q
    parts = spec.split(",")
    name, N, K, M = parts[0], int(parts[1]), int(parts[2]), int(parts[3])
    copies = int(parts[4]) if len(parts) > 4 else 4
    t = capi.GGUF_TYPES[name]
    base = torch.from_numpy(Q.random_gguf_weight(name, N, K, seed=1)).to(ctx.dev)
    weights = [base.clone() for _ in range(copies)]
    A = torch.randn(M, K, device=ctx.dev).to(torch.bfloat16)
    call = (lambda w: ops.gguf_mmq(A, w, t, N, K)) if mmq else (lambda w: ops.gguf_mmvq(A, w, t, N, K))
    for i in range(calls):
        call(weights[i % copies])
    torch.cuda.synchronize()
    nbytes = N * (K // capi.BLOCK_VALUES[t]) * capi.BLOCK_BYTES[t] + M * K * 2 + M * N * 2
    line = {"metric": "shape_probe", "config": {"workload": f"{name} {N}x{K} M={M}, {'mmq' if mmq else 'mmvq'}",
                                                "copies": copies, "calls": calls}, "n_gpus": 1}
    if timed:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for w in weights:
                call(w)
        ms = time_steps(g.replay, 20, 3, ctx) / copies
        line.update({"ms_per_call": ms, "gbps": nbytes / (ms * 1e-3) / 1e9,
                     "tflops": 2.0 * M * N * K / (ms * 1e-3) / 1e12})
    return line


# --------------------------------------------------------------------------------------
# CPU baselines: the reference's dequantize-then-matmul path (tests/test_reference.py:88-102,
# 284-329) on the host cores, bounded samples.  Only bench.py's cpu_baseline leg and its
# reference arm call these.
# --------------------------------------------------------------------------------------
def _pool_map(fn, items, threads):
    from concurrent.futures import ThreadPoolExecutor
    try:
        from threadpoolctl import threadpool_limits
    except ImportError:          # pragma: no cover - threadpoolctl ships with the image
        threadpool_limits = None
    with ThreadPoolExecutor(max_workers=threads) as ex:
        if threadpool_limits is None:
            return list(ex.map(fn, items))
        with threadpool_limits(limits=1):      # one BLAS thread per pool worker: no oversubscription
            return list(ex.map(fn, items))


def cpu_moe(tokens_sample=64, threads=None):
    """Reference-style grouped GEMM of the MoE layer on the CPU: dequantize every routed
    expert's three matrices, then matmul its rows (ref_grouped_gemm).  Timed on a sample of
    `tokens_sample` tokens with all 128 experts' weights resident; scaled per token."""
    import oracle
    from layerstormgemmkernels_b200.formats import Q4_K
    oracle.build()
    threads = threads or os.cpu_count() or 1
    E, k, H, I = MOE["E"], MOE["k"], MOE["H"], MOE["I"]
    g = torch.Generator().manual_seed(3)
    base = [(_q4k(torch.randn(I, H, generator=g) * 0.02), _q4k(torch.randn(I, H, generator=g) * 0.02),
             _q4k(torch.randn(H, I, generator=g) * 0.02)) for _ in range(8)]
    rng = np.random.default_rng(0)
    x = rng.standard_normal((tokens_sample, H)).astype(np.float32)
    logits = rng.standard_normal((tokens_sample, E)).astype(np.float32)
    top = np.argsort(-logits, axis=1)[:, :k]

    def expert(e):
        rows = np.nonzero((top == e).any(axis=1))[0]
        if rows.size == 0:
            return 0
        gw, uw, dw = (oracle.dequant(Q4_K, m) for m in base[e % 8])
        xe = x[rows]
        gt, ut = xe @ gw.T, xe @ uw.T
        act = gt / (1.0 + np.exp(-gt)) * ut
        return (act @ dw.T).shape[0]

    _pool_map(expert, range(E), threads)
    t0 = time.perf_counter()
    _pool_map(expert, range(E), threads)
    dt = time.perf_counter() - t0
    flops = 6.0 * tokens_sample * k * H * I
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "ms_sample": dt * 1e3,
            "sample": f"{tokens_sample} tokens through all routed experts (dequantize Q4_K -> fp32, matmul), "
                      f"{threads} pool threads x 1 BLAS thread; the dequantization does not shrink with the "
                      "sample, so per-token cost at 4096 tokens is lower than this figure suggests"}


def cpu_prefill(rows_sample=64, threads=None, w_full=None):
    """Dequantize the 14336x4096 Q4_K weight, then matmul `rows_sample` token rows; the matmul
    time is scaled to M rows by the caller's flops (the dequantization is paid once)."""
    import oracle
    from layerstormgemmkernels_b200.formats import Q4_K
    oracle.build()
    threads = threads or os.cpu_count() or 1
    w = prefill_weight() if w_full is None else w_full
    packed = _q4k(w)
    x = np.random.default_rng(0).standard_normal((rows_sample, 4096)).astype(np.float32)
    chunks = np.array_split(np.arange(14336), threads * 2)

    def one(idx):
        return x @ oracle.dequant(Q4_K, packed[idx[0]:idx[-1] + 1]).T

    _pool_map(one, chunks, threads)
    t0 = time.perf_counter()
    _pool_map(one, chunks, threads)
    dt = time.perf_counter() - t0
    flops = 2.0 * rows_sample * 14336 * 4096
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port", "ms_sample": dt * 1e3,
            "sample": f"{rows_sample} token rows against the whole 14336x4096 weight (dequantize -> fp32, matmul), "
                      f"{threads} pool threads x 1 BLAS thread"}


def cpu_fp8_quant(threads=None):
    """ref_dynamic_fp8_quant-style (tests/test_reference.py:56-73) on a 512 x 4096 slice."""
    x = torch.randn(512, 4096, generator=torch.Generator().manual_seed(11)).to(torch.bfloat16)
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)

    def once():
        xf = x.float().reshape(512, 32, 128)
        amax = xf.abs().amax(-1, keepdim=True).clamp_min(1e-12)
        sc = amax / 448.0
        return (xf / sc).to(torch.float8_e4m3fn), sc
    once()
    t0 = time.perf_counter()
    for _ in range(5):
        once()
    dt = (time.perf_counter() - t0) / 5
    nbytes = 512 * 4096 * 3 + 512 * 32 * 4
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": "512 x 4096 slice of the tensor, torch CPU ops, 5 repetitions"}
