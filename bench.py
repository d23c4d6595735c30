#!/usr/bin/env python
"""Benchmark of the quantized-GEMM hot path.

Headline (the JSON line on stdout): GGUF mmvq decode over one Llama-3-8B-shaped layer,
Q4_K, batch 1, in GB/s against the measured HBM peak.  A "step" is one decode pass over the
seven projections of one transformer layer (q/o 4096x4096, k/v 1024x4096, gate/up
14336x4096, down 4096x14336; weights quantized from N(0, 0.02) seed 1, activations N(0, 1)
as bf16), each projection the reference-compatible operator: Q8_1 activation quantization +
integer mat-vec.  Weights are resident in HBM; successive steps walk over several copies of
the layer (more than the 126 MB L2), captured together as one CUDA graph the way a decoder's
layers are, so that every step streams its weights from DRAM.

After the headline leg the same run measures the other cells of the metric and puts them
into the headline line as compact objects (their full lines go to stderr):
  cells     mmvq at batch 2/4/8, Q6_K, Q4_0 4096x4096
  sharded   the MoE layer (128 experts top-8, expert-parallel over the ranks, strong and weak
            scaling), the Q4_K 14336x4096 prefill GEMM (column-split over the ranks)
  nvfp4     the NVFP4 expert block (8 experts top-2, H=4096, I=14336, 4096 tokens)
  quant     the activation quantizers on a 4096x4096 tensor

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch M] [--type Q4_K|Q6_K|...]
                    [--legs all|none|cells,moe,prefill,nvfp4,quant] [--workload ...]
    python bench.py --impl reference ...   # the CPU dequantize-then-matmul path, host cores

With --gpus N > 1 (launched by torchrun) every rank runs its own replica of the decode step
(the mat-vec does not shard: "replicas only"; value is the sum) and the sharded legs run
expert-parallel / column-split over the N ranks.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time
import traceback
from types import SimpleNamespace

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LAYER = [("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096),
         ("gate", 14336, 4096), ("up", 14336, 4096), ("down", 4096, 14336)]
GROUP = {"q": 0, "k": 0, "v": 0, "o": 1, "gate": 2, "up": 2, "down": 3}
L2_BYTES = 126 * 1024 * 1024


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def algorithmic_bytes(type_name, M, layer=LAYER):
    """Packed weight bytes + bf16 activations read once + bf16 outputs, per step."""
    from layerstormgemmkernels_b200.formats import GGUF_TYPES, BLOCK_BYTES, BLOCK_VALUES
    t = GGUF_TYPES[type_name]
    return sum(N * (K // BLOCK_VALUES[t]) * BLOCK_BYTES[t] + M * K * 2 + M * N * 2 for _, N, K in layer)


def make_layer_weights(type_name, seed=1, threads=None, layer=LAYER):
    """Packed weights of one layer, quantized from N(0, 0.02) (host, numpy)."""
    import torch
    from concurrent.futures import ThreadPoolExecutor
    from layerstormgemmkernels_b200 import quantize as Q
    fn = Q.QUANTIZERS[type_name]
    threads = threads or os.cpu_count() or 4
    out = []
    g = torch.Generator().manual_seed(seed)
    with ThreadPoolExecutor(max_workers=threads) as ex:
        for _, N, K in layer:
            w = (torch.randn(N, K, generator=g) * 0.02).numpy()
            chunks = np.array_split(np.arange(N), min(N, threads * 4))
            parts = list(ex.map(lambda idx: fn(w[idx[0]:idx[-1] + 1]), chunks))
            out.append(np.concatenate(parts, axis=0))
    return out


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            parts = [p.strip() for p in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------------------
# CPU arm: the reference's dequantize-then-matmul path on the host cores
# ----------------------------------------------------------------------------------------
def cpu_reference_step(type_name, weights, x_f32, threads, layer=LAYER):
    """The reference's CPU path for this metric: dequantize the packed weight to fp32, then
    matmul (tests/test_reference.py: ref_q4k_dequant + ref_q4k_gemm, :284-329), here through
    the C oracle's block decoders; row slices spread over `threads` pool workers, each with
    ONE BLAS thread (a multi-threaded BLAS inside every worker oversubscribes the cores)."""
    import oracle
    from bench_workloads import _pool_map
    from layerstormgemmkernels_b200.formats import GGUF_TYPES
    t = GGUF_TYPES[type_name]

    def one(args):
        W, x = args
        return x @ oracle.dequant(t, W).T

    outs = []
    for W, (_, N, K) in zip(weights, layer):
        x = x_f32[K]
        chunks = np.array_split(np.arange(N), min(N, threads * 2))
        parts = _pool_map(one, [(W[idx[0]:idx[-1] + 1], x) for idx in chunks], threads)
        outs.append(np.concatenate(parts, axis=1))
    return outs


def cpu_decode_baseline(type_name, M, host_w, repeats=2):
    import oracle
    oracle.build()
    threads = os.cpu_count() or 1
    rng = np.random.default_rng(0)
    xf = {K: rng.standard_normal((M, K)).astype(np.float32) for K in (4096, 14336)}
    cpu_reference_step(type_name, host_w, xf, threads)
    t0 = time.perf_counter()
    for _ in range(repeats):
        cpu_reference_step(type_name, host_w, xf, threads)
    dt = (time.perf_counter() - t0) / repeats
    abytes = algorithmic_bytes(type_name, M)
    return {"value": abytes / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "threads": f"{threads} pool threads x 1 BLAS thread", "ms_per_step": dt * 1e3,
            "sample": f"{repeats} whole-layer steps (7 projections each) after 1 warm-up"}


def run_reference(args, rank):
    """--impl reference: the CPU path on the host cores (rank 0 only), same config and metric."""
    if rank != 0:
        return
    import bench_workloads as W
    steps = min(args.steps, 5)
    base = {"impl": "reference", "n_gpus": args.gpus, "steps": steps, "warmup": 1, "higher_is_better": True,
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "gpu_launches": 0}
    if args.workload in ("decode", "mmvq"):
        host_w = make_layer_weights(args.type)
        cb = cpu_decode_baseline(args.type, args.batch, host_w, repeats=steps)
        line = dict(base, metric=f"{args.type.lower()}_mmvq_gbps", value=cb["value"], unit="GB/s",
                    ms_per_step=cb["ms_per_step"], scaling="weak", config=workload_config(args), cpu_baseline=cb)
    elif args.workload == "moe":
        cb = W.cpu_moe(tokens_sample=64)
        line = dict(base, metric="moe_grouped_gemm_tflops", value=cb["value"], unit="TFLOP/s",
                    ms_per_step=cb["ms_sample"], scaling="strong",
                    config={"workload": "MoE layer, 128 experts top-8, H=2048, I=768, Q4_K (64-token sample)"},
                    cpu_baseline=cb)
    elif args.workload == "prefill":
        cb = W.cpu_prefill(rows_sample=64)
        line = dict(base, metric="q4_k_mmq_prefill_tflops", value=cb["value"], unit="TFLOP/s",
                    ms_per_step=cb["ms_sample"], scaling="strong",
                    config={"workload": "Q4_K 14336x4096 prefill GEMM (64-row sample)"}, cpu_baseline=cb)
    else:
        print(json.dumps({"impl": "reference", "unavailable":
                          f"no CPU arm for --workload {args.workload}"}), flush=True)
        return
    line["e2e"] = {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    print(json.dumps(line), flush=True)


def workload_config(args):
    return {"workload": f"llama3-8b layer decode, {args.type} mmvq, batch {args.batch}: "
                        "q,k,v,o,gate,up,down",
            "type": args.type, "batch": args.batch,
            "shapes": {n: [N, K] for n, N, K in LAYER},
            "l2_defeat": "steps walk over layer copies totalling more than 2.5x the 126 MB L2",
            "launch": "one CUDA graph over all layer copies (a decoder's layers back to back), each layer one "
                      "lsg_gguf_mmvq_batch call over the seven projections, which have four distinct inputs and "
                      "no dependency on each other inside the call: the library runs the six K = 4096 projections "
                      "as one launch and down as a second one that does not wait for the first; activations "
                      "quantized inside the launches (above 32768 values: a quantizer launch per input, one "
                      "launch per input, each waiting for the one before)",
            "parallelism": "replicas only"}


# ----------------------------------------------------------------------------------------
# The decode layer on the GPU
# ----------------------------------------------------------------------------------------
def planned_launches(capi, arr, n):
    """(mat-vec launches, all kernel launches) of one lsg_gguf_mmvq_batch call over `arr[:n]`, asked
    of lsg_gguf_mmvq_batch_plan: a mat-vec whose activations are above the in-kernel
    quantizer's limit has a quantizer launch in front of it (kind + 4)."""
    kind = (ctypes.c_int * max(n, 1))()
    groups = capi.lib.lsg_gguf_mmvq_batch_plan(arr, n, None, None, kind, n)
    if groups < 0:
        raise RuntimeError("lsg_gguf_mmvq_batch_plan failed")
    return groups, sum(2 if kind[i] >= 4 else 1 for i in range(groups))


class DecodeLayerBench:
    """Device-resident layer copies, their argument blocks and graphs."""

    def __init__(self, type_name, M, dev, host_w=None, layer=LAYER, group=GROUP, min_copies=2):
        import torch
        from layerstormgemmkernels_b200 import capi
        self.torch, self.capi = torch, capi
        self.M, self.dev, self.layer, self.group = M, dev, layer, group
        self.t = capi.GGUF_TYPES[type_name]
        self.host_w = host_w if host_w is not None else make_layer_weights(type_name, layer=layer)
        layer_bytes = sum(w.nbytes for w in self.host_w)
        self.copies = max(min_copies, int(2.5 * L2_BYTES // layer_bytes) + 1)
        self.layers = [[torch.from_numpy(w).to(dev) for w in self.host_w] for _ in range(self.copies)]
        g = torch.Generator().manual_seed(0)
        # the distinct inputs of a decoder layer: the attention input (q, k, v), the attention
        # output (o), the MLP input (gate, up) and the gated product (down)
        self.xin = {}
        for name, _, K in layer:
            if group[name] not in self.xin:
                self.xin[group[name]] = torch.randn(M, K, generator=g).to(torch.bfloat16).pin_memory()
        self.x_dev = {k: v.to(dev) for k, v in self.xin.items()}
        self.outs = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for _, N, _ in layer]
        self.abytes = algorithmic_bytes(type_name, M, layer)
        self.args = [self._params(w) for w in self.layers]
        need = capi.lib.lsg_gguf_mmvq_batch_workspace_bytes(self.args[0], len(layer))
        self.ws = torch.empty((max(need, 256),), dtype=torch.uint8, device=dev)
        # launches of one lsg_gguf_mmvq_batch call, as the library's own planner forms them
        try:
            self.n_matvec, self.launches_per_step = planned_launches(capi, self.args[0], len(layer))
        except Exception:  # noqa: BLE001 - an older library without the planner: its rule restated
            runs = []
            for name, _, K in layer:
                fused = M * K <= 32768
                if runs and runs[-1][1] == K and runs[-1][2] < 6 and (runs[-1][0] == group[name] or (fused and runs[-1][3])):
                    runs[-1][2] += 1
                    runs[-1][0] = group[name]
                else:
                    runs.append([group[name], K, 1, fused])
            self.n_matvec = len(runs)
            self.launches_per_step = sum(1 if f else 2 for _, _, _, f in runs)

    def _params(self, weights):
        capi = self.capi
        arr = (capi.GgufMmvqParams * len(self.layer))()
        for i, (W, out, (name, N, K)) in enumerate(zip(weights, self.outs, self.layer)):
            arr[i] = capi.GgufMmvqParams(M=self.M, N=N, K=K, A=self.x_dev[self.group[name]].data_ptr(),
                                         B=W.data_ptr(), C=out.data_ptr(), type=self.t, out_dtype=capi.DTYPE_BF16)
        return arr

    def step(self, arr):
        st = ctypes.c_void_p(self.torch.cuda.current_stream().cuda_stream)
        self.capi.check(self.capi.lib.lsg_gguf_mmvq_batch(arr, len(self.layer), ctypes.c_void_p(self.ws.data_ptr()),
                                                          self.ws.numel(), st))

    def capture(self):
        torch = self.torch
        for arr in self.args:
            self.step(arr)
        torch.cuda.synchronize()
        self.all_graph = torch.cuda.CUDAGraph()          # every layer copy back to back
        with torch.cuda.graph(self.all_graph):
            for arr in self.args:
                self.step(arr)
        self.one_graphs = []                             # single layers, for a remainder of steps
        for arr in self.args:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.step(arr)
            self.one_graphs.append(g)

    def run_steps(self, n):
        full, rest = divmod(n, self.copies)
        for _ in range(full):
            self.all_graph.replay()
        for i in range(rest):
            self.one_graphs[i].replay()

    def time(self, steps, warmup, world, dist=None, sampler=None):
        torch = self.torch
        self.run_steps(max(warmup, self.copies))
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        if sampler is not None:
            sampler.start()
            time.sleep(0.15)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        self.run_steps(steps)
        e1.record()
        torch.cuda.synchronize()
        ms_total = e0.elapsed_time(e1)
        clocks = sampler.stop() if sampler is not None else None
        if world > 1:
            tt = torch.tensor([ms_total], device=self.dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms_total = float(tt.item())
        return ms_total / steps, clocks


def decode_cell(type_name, M, dev, steps, warmup, layer=LAYER, group=GROUP):
    """One secondary mmvq cell (other batch sizes, other types): ms/step, GB/s, fraction."""
    b = DecodeLayerBench(type_name, M, dev, layer=layer, group=group)
    b.capture()
    ms, _ = b.time(steps, warmup, 1)
    peak, _ = load_peaks()
    gbs = b.abytes / (ms * 1e-3) / 1e9
    return {"ms_per_step": ms, "gbps": gbs, "frac_of_hbm_peak": gbs / peak, "launches_per_step": b.launches_per_step,
            "algorithmic_bytes": b.abytes}


def compact(line):
    """The fields of a secondary line that go into the headline line."""
    if line is None:
        return None
    if "error" in line:
        return {"error": line["error"]}
    out = {"value": line.get("value"), "unit": line.get("unit"), "ms_per_step": line.get("ms_per_step"),
           "scaling": line.get("scaling"), "n_gpus": line.get("n_gpus")}
    if "roofline" in line:
        out["frac"] = line["roofline"].get("frac")
        out["bound"] = line["roofline"].get("bound")
    for k in ("expert_block", "equal_to_nccl_exchange", "equal_to_nccl_gather", "overflow", "cells", "cpu_baseline"):
        if k in line and line[k] is not None:
            out[k] = line[k]
    if "config" in line:
        out["parallelism"] = line["config"].get("parallelism")
        out["workload"] = line["config"].get("workload")
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--type", default="Q4_K", choices=["Q4_K", "Q6_K", "Q8_0", "Q4_0"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="decode",
                    choices=["decode", "mmvq", "moe", "prefill", "nvfp4", "quant", "shape"],
                    help="decode (default; `mmvq` is the same): the headline layer plus the legs of --legs; "
                         "moe / prefill / nvfp4 / quant: that workload alone as the stdout line; "
                         "shape: one --shape for profilers")
    ap.add_argument("--legs", default="all", help="secondary legs after the headline: all, none, or a comma list of "
                                                  "cells,moe,prefill,nvfp4,quant")
    ap.add_argument("--tokens", type=int, default=4096, help="tokens (moe, nvfp4) or rows M (prefill)")
    ap.add_argument("--ep", default="peer", choices=["peer", "nccl"],
                    help="several GPUs: exchange rows by peer-memory stores or by NCCL collectives")
    ap.add_argument("--weak", action="store_true", help="moe: --tokens is per GPU (weak scaling)")
    ap.add_argument("--ep-groups", type=int, default=1, help="moe on several GPUs: groups of local experts pipelined on side streams (1: none)")
    ap.add_argument("--ep-chunks", type=int, default=1, help="moe on several GPUs: pipelined token halves of the peer exchange (1: none)")
    ap.add_argument("--shape", default="Q4_K,14336,4096,1,8", help="shape mode: TYPE,N,K,M[,COPIES]")
    ap.add_argument("--calls", type=int, default=12, help="shape mode: calls issued before timing")
    ap.add_argument("--mmq", action="store_true", help="shape mode: the tensor-core GEMM instead of the mat-vec")
    ap.add_argument("--no-time", action="store_true", help="shape mode: only issue the calls (profiler runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    from layerstormgemmkernels_b200 import capi, ops  # raises if the CUDA library is missing
    import bench_workloads as W

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ctx = SimpleNamespace(rank=rank, world=world, dev=dev, local_rank=local_rank)
    sec_steps = max(3, min(args.steps, 50))
    sec_warm = max(3, min(args.warmup, 5))

    def finish(line):
        status = capi.device_status()
        if status not in (0,):
            line["device_status"] = status
        if rank == 0:
            print(json.dumps(line), flush=True)
        if world > 1:
            dist.destroy_process_group()
        if status != 0:
            raise SystemExit(f"a kernel reported device status {status} (a wait that ran out, or an overflow)")

    # ---- single-workload modes ------------------------------------------------------
    if args.workload == "shape":
        finish(W.run_shape(ctx, args.shape, args.calls, mmq=args.mmq, timed=not args.no_time))
        return
    if args.workload in ("moe", "prefill", "nvfp4", "quant"):
        sampler = ClockSampler(local_rank)
        sampler.start()
        if args.workload == "moe":
            line = W.run_moe(ctx, args.tokens, sec_steps, sec_warm, weak=args.weak, ep=args.ep, chunks=args.ep_chunks, groups=args.ep_groups)
            if world == 1 and not args.no_cpu_baseline:
                line["cpu_baseline"] = W.cpu_moe()
        elif args.workload == "prefill":
            line = W.run_prefill(ctx, args.tokens, sec_steps, sec_warm, ep=args.ep)
            if world == 1 and not args.no_cpu_baseline:
                line["cpu_baseline"] = W.cpu_prefill()
        elif args.workload == "nvfp4":
            line = W.run_nvfp4(ctx, args.tokens, sec_steps, sec_warm)
        else:
            line = W.run_quant(ctx, sec_steps, sec_warm)
            if world == 1 and not args.no_cpu_baseline:
                line["cpu_baseline"] = W.cpu_fp8_quant()
        line["clocks"] = sampler.stop()
        finish(line)
        return

    # ---- headline: the decode layer ------------------------------------------------------
    M = args.batch
    bench = DecodeLayerBench(args.type, M, dev)
    bench.capture()
    ms_per_step, clocks = bench.time(args.steps, args.warmup, world, dist, ClockSampler(local_rank))
    abytes = bench.abytes
    value = world * abytes / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the operator API, host buffers --------------------------
    e2e_steps = min(args.steps, 400)
    t = bench.t
    res_host = [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for _, N, _ in LAYER]
    # one prepared batch per layer copy: pointers only; every run reads the activations from
    # page-locked host memory and writes the results there; all copies captured as one graph
    batches = [ops.HostMmvqBatch([(bench.xin[GROUP[name]], Wt, t, N, K, res)
                                  for Wt, res, (name, N, K) in zip(weights, res_host, LAYER)])
               for weights in bench.layers]
    for bt in batches:
        bt.enqueue()
    torch.cuda.synchronize()
    e2e_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(e2e_graph):
        for bt in batches:
            bt.enqueue()
    for bt in batches:
        bt.capture()

    def e2e_steps_run(n):
        full, rest = divmod(n, bench.copies)
        for _ in range(full):
            e2e_graph.replay()
        for i in range(rest):
            batches[i].run()

    e2e_steps_run(2 * bench.copies)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_steps_run(e2e_steps)
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    if world > 1:
        tt = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms = float(tt.item())
    e2e_value = world * abytes / (e2e_ms * 1e-3) / 1e9
    h2d = sum(v.numel() * 2 for v in bench.xin.values())
    d2h = sum(M * N * 2 for _, N, _ in LAYER)

    peak, peak_kind = load_peaks()
    n_gemv = bench.n_matvec
    achieved = (abytes / n_gemv) / (ms_per_step * 1e-3 / n_gemv) / 1e9
    line = {
        "metric": f"{args.type.lower()}_mmvq_gbps", "value": value, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic", "config": workload_config(args),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": f"{peak_kind} (copy bandwidth)",
                     "traffic": None, "algorithmic_bytes_per_step": abytes,
                     "launches_per_step": bench.launches_per_step},
        "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "api": "layerstormgemmkernels_b200.ops.HostMmvqBatch (lsg_gguf_mmvq_host_batch, all layer copies "
                       "captured as one CUDA graph): the seven projections of a layer, page-locked host tensors "
                       "in and out"},
        "gpu_launches": args.steps * bench.launches_per_step,
        "clocks": clocks,
    }
    traffic_file = os.path.join(ROOT, "profiles", "traffic.txt")
    if os.path.exists(traffic_file):
        with open(traffic_file) as f:
            for ln in f:
                parts = ln.split()
                if len(parts) == 2 and parts[0] == f"{args.type}_M{M}":
                    line["roofline"]["traffic"] = int(parts[1])

    # ---- secondary legs -----------------------------------------------------------------
    legs = set() if args.legs == "none" else (
        {"cells", "moe", "prefill", "nvfp4", "quant"} if args.legs == "all" else set(args.legs.split(",")))
    host_w = bench.host_w
    del bench, batches, e2e_graph
    torch.cuda.empty_cache()

    def leg(name, fn):
        """Runs one secondary leg; a failure is recorded in its object, never fatal to the line.
        Under torchrun every rank must take the same path, so errors are not swallowed there."""
        try:
            res = fn()
        except Exception as exc:   # noqa: BLE001
            if world > 1:
                raise
            traceback.print_exc(file=sys.stderr)
            res = {"error": f"{type(exc).__name__}: {exc}"}
        if rank == 0 and isinstance(res, dict) and "metric" in res:
            print("SECONDARY " + json.dumps(res), file=sys.stderr, flush=True)
        torch.cuda.empty_cache()
        return res

    if "cells" in legs and world == 1:
        cells = {}
        cell_steps = max(4, min(args.steps, 200))
        for m in (2, 4, 8):
            cells[f"{args.type}_batch{m}"] = leg(f"batch{m}", lambda m=m: decode_cell(args.type, m, dev, cell_steps, 8))
        other = "Q6_K" if args.type == "Q4_K" else "Q4_K"
        cells[f"{other}_batch1"] = leg(other, lambda: decode_cell(other, 1, dev, cell_steps, 8))
        # the reference's own CPU-runnable case: one Q4_0 4096 x 4096 mat-vec
        cells["Q4_0_4096x4096_batch1"] = leg("q4_0", lambda: decode_cell(
            "Q4_0", 1, dev, cell_steps, 8, layer=[("w", 4096, 4096)], group={"w": 0}))
        line["cells"] = cells
    sharded = {}
    if "moe" in legs:
        sharded["moe"] = compact(leg("moe", lambda: W.run_moe(ctx, 4096, sec_steps, sec_warm, ep=args.ep)))
        if world > 1:
            sharded["moe_weak"] = compact(leg("moe_weak", lambda: W.run_moe(ctx, 4096, sec_steps, sec_warm, weak=True,
                                                                          ep=args.ep, check=False)))
        else:
            for tk in (64, 1):
                sharded[f"moe_tokens{tk}"] = compact(leg(f"moe{tk}", lambda tk=tk: W.run_moe(ctx, tk, sec_steps, sec_warm)))
    if "prefill" in legs:
        w_full = W.prefill_weight()
        sharded["prefill_m4096"] = compact(leg("prefill", lambda: W.run_prefill(ctx, 4096, sec_steps, sec_warm,
                                                                                ep=args.ep, w_full=w_full)))
        if world == 1:
            sharded["prefill_m512"] = compact(leg("prefill512", lambda: W.run_prefill(ctx, 512, sec_steps, sec_warm,
                                                                                      w_full=w_full)))
        del w_full
    if sharded:
        line["sharded"] = sharded
    if "nvfp4" in legs and 8 % world == 0:
        line["nvfp4"] = compact(leg("nvfp4", lambda: W.run_nvfp4(ctx, 4096, max(3, min(sec_steps, 10)), 3)))
    if "quant" in legs and world == 1:
        line["quant"] = compact(leg("quant", lambda: W.run_quant(ctx, sec_steps, sec_warm)))

    # ---- CPU baselines beside the numbers (rank 0, one GPU) -------------------------------
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_decode_baseline(args.type, M, host_w)
        if "moe" in legs and isinstance(sharded.get("moe"), dict):
            sharded["moe"]["cpu_baseline"] = leg("cpu_moe", W.cpu_moe)
        if "prefill" in legs and isinstance(sharded.get("prefill_m4096"), dict):
            sharded["prefill_m4096"]["cpu_baseline"] = leg("cpu_prefill", W.cpu_prefill)
        if "quant" in legs and isinstance(line.get("quant"), dict):
            line["quant"]["cpu_baseline"] = leg("cpu_quant", W.cpu_fp8_quant)
    finish(line)


if __name__ == "__main__":
    main()
