"""Secondary benchmark workloads behind `bench.py --workload moe|prefill` (same JSON line as
the headline workload): the expert-parallel MoE layer and the column-split prefill GEMM.
"""
import json
import sys
import os
import time

import numpy as np
import torch
import torch.distributed as dist

from . import capi, ops, quantize as Q, distributed as D

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _peak_tflops():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["bf16_tflops_sustained"]), "measured (cuBLAS bf16, sustained)"
    return 1400.0, "fallback"


def _time_steps(step, steps, warmup, world, dev, sampler=None):
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.start()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    if sampler is not None:
        _CLOCKS.update(sampler.stop())
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps


_CLOCKS = {}


def run(args, rank, local_rank, world, sampler_cls=None):
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    steps = min(args.steps, 200)
    warmup = max(3, min(args.warmup, 10))
    sampler = sampler_cls(local_rank) if sampler_cls is not None else None
    if args.workload == "moe":
        line = _moe(args, rank, world, dev, steps, warmup, sampler)
    else:
        line = _prefill(args, rank, world, dev, steps, warmup, sampler)
    line["clocks"] = dict(_CLOCKS) if _CLOCKS else None
    line["cpu_baseline"] = None   # the CPU reference arm is timed on the headline workload only
    status = capi.device_status()
    if status != 0:
        raise SystemExit(f"a kernel reported a timed-out device-side wait (code {status})")
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _moe(args, rank, world, dev, steps, warmup, sampler=None):
    E, k, H, I = 128, 8, 2048, 768
    weak = bool(getattr(args, "weak", False))
    T_total = args.tokens * world if weak else args.tokens
    if T_total % world != 0:
        raise SystemExit("--tokens must be divisible by the number of GPUs")
    T = T_total // world                       # strong scaling splits the batch, weak keeps it per GPU
    t = capi.Q4_K
    e0, e1 = D.expert_range(rank, world, E)
    # eight distinct experts quantized from N(0, 0.02) seed 3, tiled over the rank's experts
    g = torch.Generator().manual_seed(3)
    base = []
    for _ in range(8):
        base.append((Q.quantize_q4_k((torch.randn(I, H, generator=g) * 0.02).numpy()),
                     Q.quantize_q4_k((torch.randn(I, H, generator=g) * 0.02).numpy()),
                     Q.quantize_q4_k((torch.randn(H, I, generator=g) * 0.02).numpy())))
    gate_w = [torch.from_numpy(base[e % 8][0]).to(dev) for e in range(e0, e1)]
    up_w = [torch.from_numpy(base[e % 8][1]).to(dev) for e in range(e0, e1)]
    down_w = [torch.from_numpy(base[e % 8][2]).to(dev) for e in range(e0, e1)]
    ptr = lambda ws: torch.tensor([w.data_ptr() for w in ws], dtype=torch.int64, device=dev)
    gate_p, up_p, down_p = ptr(gate_w), ptr(up_w), ptr(down_w)
    gg = torch.Generator().manual_seed(1000 + rank)
    hidden = torch.randn(T, H, generator=gg).to(torch.bfloat16).to(dev)
    logits = torch.randn(T, E, generator=gg).to(dev)
    hidden_host = hidden.cpu().pin_memory()
    logits_host = logits.cpu().pin_memory()

    def ffn(rows, offs):
        return ops.gguf_moe_ffn(rows, offs, gate_p, up_p, down_p, t, H, I)

    # Exchange between the ranks: stores into the peers' buffers (default), or the NCCL
    # all-to-all pair when symmetric memory cannot be set up (or with --ep nccl).
    exchange = None
    ep_mode = "single"
    if world > 1:
        ep_mode = getattr(args, "ep", "peer")
        if ep_mode == "peer":
            try:
                exchange = D.EpPeerExchange.make(E, k, H, T)
            except Exception as exc:   # noqa: BLE001 - any failure of the optional path falls back
                if rank == 0:
                    print(f"peer-memory exchange unavailable ({type(exc).__name__}: {exc}); using NCCL all-to-all",
                          file=sys.stderr)
                ep_mode = "nccl"

    def layer(h, lg):
        if world == 1:
            idx, w = ops.moe_route(lg, k)
            offs, perm, inv = ops.moe_permutation(idx, E)
            return ops.moe_unpermute(ffn(ops.moe_permute(h, perm, k), offs), inv, w)
        if exchange is not None:
            return exchange.layer(h, lg, ffn, ops.moe_route, ops.moe_permutation, ops.moe_unpermute)
        return D.ep_moe_layer(h, lg, k, E, ffn, ops.moe_route, ops.moe_permutation, ops.moe_permute,
                              ops.moe_unpermute)

    ms = _time_steps(lambda: layer(hidden, logits), steps, warmup, world, dev, sampler)
    if exchange is not None and exchange.overflowed():
        raise SystemExit("expert-parallel receive buffer overflowed (raise the capacity factor)")
    # the expert block alone (the grouped GEMMs with their operand preparation) on this rank's
    # routed rows, single GPU only: what the tensor-pipe roofline is about
    gemm_ms = None
    if world == 1:
        idx, _w = ops.moe_route(logits, k)
        offs, perm, _inv = ops.moe_permutation(idx, E)
        rows = ops.moe_permute(hidden, perm, k)
        gemm_ms = _time_steps(lambda: ffn(rows, offs), steps, warmup, world, dev)

    def e2e_step():
        h = hidden_host.to(dev, non_blocking=True)
        lg = logits_host.to(dev, non_blocking=True)
        return layer(h, lg).cpu()
    e2e_ms = _time_steps(e2e_step, min(steps, 20), 3, world, dev)

    flops = 6.0 * T_total * k * H * I
    peak, kind = _peak_tflops()
    value = flops / (ms * 1e-3) / 1e12
    return {
        "metric": "moe_grouped_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak" if weak else "strong", "vs_baseline": None, "dtype": "f16 (tcgen05, fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": f"MoE layer, 128 experts top-8, H=2048, I=768, Q4_K, {T_total} tokens: "
                               "route, permute, gate/up/down grouped GEMMs, SwiGLU, combine",
                   "tokens": T_total,
                   "parallelism": (f"ep{world}, rows exchanged by peer-memory stores" if ep_mode == "peer"
                                   else f"ep{world}, NCCL all-to-all" if world > 1 else "single"),
                   "l2_defeat": "339 MB of expert weights per rank set exceed the 126 MB L2"},
        "roofline": {"bound": "tensor", "achieved": value / world, "peak": peak, "unit": "TFLOP/s",
                     "frac": value / world / peak, "peak_kind": kind, "traffic": None,
                     "note": "whole layer (routing, permute, expert block, combine) over the GEMM flops"},
        "expert_block": None if gemm_ms is None else {
            "what": "lsg_gguf_moe_ffn alone on the routed rows: operand preparation, gate|up GEMM, SwiGLU, down GEMM",
            "ms": gemm_ms, "tflops": flops / (gemm_ms * 1e-3) / 1e12,
            "frac_of_peak": flops / (gemm_ms * 1e-3) / 1e12 / peak},
        "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": T * H * 2 + T * E * 4, "d2h_bytes_per_step": T * H * 2},
        # library kernels per step and rank: route, 3 x permutation, gather, tile map, activation
        # preparation, gate|up GEMM, SwiGLU preparation, down GEMM, combine
        "gpu_launches": steps * 11,
    }


def _prefill(args, rank, world, dev, steps, warmup, sampler=None):
    N, K, M = 14336, 4096, args.tokens
    t = capi.Q4_K
    n0, n1 = D.column_slab(rank, world, N)
    g = torch.Generator().manual_seed(2)
    w = (torch.randn(N, K, generator=g) * 0.02).numpy()
    slab = torch.from_numpy(Q.quantize_q4_k(w[n0:n1])).to(dev)
    A = torch.randn(M, K, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(dev)
    A_host = A.cpu().pin_memory()

    # Several GPUs: the all-gather is fused into the GEMM's epilogue (peer-memory stores), or,
    # with --ep nccl or when symmetric memory cannot be set up, a separate NCCL all-gather.
    fused_gather = None
    if world > 1 and getattr(args, "ep", "peer") == "peer":
        try:
            fused_gather = D.ColumnSplitPeer(M, N)
        except Exception as exc:   # noqa: BLE001 - the optional path falls back
            if rank == 0:
                print(f"peer-memory gather unavailable ({type(exc).__name__}: {exc}); using NCCL all-gather",
                      file=sys.stderr)

    def step(a=A):
        if fused_gather is not None:
            return fused_gather.gemm(a, slab, t, K)
        out = ops.gguf_mmq(a, slab, t, n1 - n0, K)
        return out if world == 1 else D.column_split_gather(out)

    ms = _time_steps(step, steps, warmup, world, dev, sampler)
    e2e_ms = _time_steps(lambda: step(A_host.to(dev, non_blocking=True)).cpu(), min(steps, 10), 3, world, dev)
    flops = 2.0 * M * N * K
    peak, kind = _peak_tflops()
    value = flops / (ms * 1e-3) / 1e12
    return {
        "metric": "q4_k_mmq_prefill_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16 (tcgen05, fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": f"Q4_K 14336x4096 prefill GEMM, M={M}, Q8_1 activations",
                   "parallelism": ("single" if world == 1 else
                                   f"column-split x{world}, all-gather fused into the GEMM epilogue (peer stores)"
                                   if fused_gather is not None else f"column-split x{world} + NCCL all-gather"),
                   "l2_defeat": "operands (fp16 weights 117 MB + outputs 117 MB at M=4096) exceed L2"},
        "roofline": {"bound": "tensor", "achieved": value / world, "peak": peak, "unit": "TFLOP/s",
                     "frac": value / world / peak, "peak_kind": kind, "traffic": None},
        "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2},
        # activation preparation + GEMM, plus the weight expansion pass above 2048 rows
        "gpu_launches": steps * (3 if M > 2048 else 2),
    }
