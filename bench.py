#!/usr/bin/env python
"""Headline benchmark: GGUF mmvq decode over one Llama-3-8B-shaped layer.

Metric (BASELINE.json): Q4_K mmvq GB/s against the HBM peak.  A "step" is one decode
pass of the hot path over the seven projections of one transformer layer
(q/o 4096x4096, k/v 1024x4096, gate/up 14336x4096, down 4096x14336; Q4_K weights
quantized from N(0, 0.02) seed 1, activations N(0, 1) as bf16), each projection being
one call of the reference-compatible operator: Q8_1 activation quantizer + integer
mat-vec.  Weights are resident in HBM; successive steps walk over several copies of the
layer (more than the 126 MB L2) so that every step streams its weights from DRAM.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch M] [--type Q4_K|Q6_K]
    python bench.py --impl reference ...   # the CPU dequant-then-matmul path, host cores

Prints ONE JSON line (rank 0).  With --gpus N > 1 every rank runs its own replica of the
step on its own GPU (decode mat-vec does not shard: "replicas only"); value is the sum.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LAYER = [("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096),
         ("gate", 14336, 4096), ("up", 14336, 4096), ("down", 4096, 14336)]
L2_BYTES = 126 * 1024 * 1024


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def algorithmic_bytes(type_name, M):
    """Packed weight bytes + bf16 activations read once + bf16 outputs, per step."""
    from layerstormgemmkernels_b200.capi import GGUF_TYPES, BLOCK_BYTES, BLOCK_VALUES
    t = GGUF_TYPES[type_name]
    total = 0
    for _, N, K in LAYER:
        total += N * (K // BLOCK_VALUES[t]) * BLOCK_BYTES[t] + M * K * 2 + M * N * 2
    return total


def make_layer_weights(type_name, seed=1, threads=None):
    """Packed weights of one layer, quantized from N(0, 0.02) (host, numpy)."""
    import torch
    from concurrent.futures import ThreadPoolExecutor
    from layerstormgemmkernels_b200 import quantize as Q
    fn = Q.QUANTIZERS[type_name]
    threads = threads or os.cpu_count() or 4
    out = []
    g = torch.Generator().manual_seed(seed)
    with ThreadPoolExecutor(max_workers=threads) as ex:
        for _, N, K in LAYER:
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


def cpu_reference_step(type_name, weights, x_f32, threads):
    """The reference's CPU path for this metric: dequantize the packed weight to fp32,
    then matmul (tests/test_reference.py: ref_q4k_dequant + ref_q4k_gemm, :284-329),
    here through the C oracle's block decoders, row slices spread over host threads."""
    import oracle
    from concurrent.futures import ThreadPoolExecutor
    from layerstormgemmkernels_b200.capi import GGUF_TYPES
    t = GGUF_TYPES[type_name]

    def one(args):
        W, x = args
        return x @ oracle.dequant(t, W).T

    outs = []
    with ThreadPoolExecutor(max_workers=threads) as ex:
        for W, (_, N, K) in zip(weights, LAYER):
            x = x_f32[K]
            chunks = np.array_split(np.arange(N), min(N, threads * 2))
            parts = list(ex.map(one, [(W[idx[0]:idx[-1] + 1], x) for idx in chunks]))
            outs.append(np.concatenate(parts, axis=1))
    return outs


def run_reference(args, rank, world):
    """--impl reference: the CPU dequant-then-matmul path on the host cores (rank 0 only)."""
    if rank != 0:
        return
    import oracle
    oracle.build()
    threads = os.cpu_count() or 1
    M = args.batch
    weights = make_layer_weights(args.type, threads=threads)
    rng = np.random.default_rng(0)
    x = {K: rng.standard_normal((M, K)).astype(np.float32) for K in (4096, 14336)}
    abytes = algorithmic_bytes(args.type, M)
    for _ in range(args.warmup):
        cpu_reference_step(args.type, weights, x, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_reference_step(args.type, weights, x, threads)
    dt = (time.perf_counter() - t0) / args.steps
    value = abytes / dt / 1e9
    line = {
        "impl": "reference", "metric": f"{args.type.lower()}_mmvq_gbps", "value": value,
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": "whole layer (7 projections), every step"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args):
    return {"workload": f"llama3-8b layer decode, {args.type} mmvq, batch {args.batch}: "
                        "q,k,v,o,gate,up,down",
            "type": args.type, "batch": args.batch,
            "shapes": {n: [N, K] for n, N, K in LAYER},
            "l2_defeat": "steps rotate over layer copies totalling more than the 126 MB L2",
            "launch": "one CUDA graph per layer copy of one lsg_gguf_mmvq_batch call: (q,k,v), o, (gate,up), down as four mat-vec launches, activations quantized inside them or by a quantizer launch",
            "parallelism": "replicas only"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--type", default="Q4_K", choices=["Q4_K", "Q6_K", "Q8_0", "Q4_0"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="mmvq", choices=["mmvq", "moe", "prefill"],
                    help="mmvq: the headline decode layer (default); moe: expert-parallel grouped "
                         "GEMM layer (128 experts, top-8, H=2048, I=768, Q4_K); prefill: Q4_K "
                         "14336x4096 GEMM, column-split across ranks")
    ap.add_argument("--tokens", type=int, default=4096, help="tokens (moe) or rows M (prefill)")
    ap.add_argument("--ep", default="peer", choices=["peer", "nccl"],
                    help="moe on several GPUs: exchange rows by peer-memory stores or by NCCL all-to-all")
    ap.add_argument("--weak", action="store_true",
                    help="moe: --tokens is per GPU (weak scaling) instead of the whole batch")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.workload != "mmvq":
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable":
                                  "the CPU reference arm is implemented for the headline mmvq workload only"}))
            return
        from layerstormgemmkernels_b200 import bench_extra
        bench_extra.run(args, rank, local_rank, world, ClockSampler)
        return

    if args.impl == "reference":
        if args.steps > 5:
            args.steps = 5          # each step is seconds of host work
        args.warmup = min(args.warmup, 1) if args.warmup else 0
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from layerstormgemmkernels_b200 import capi, ops  # raises if the CUDA library is missing

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    M = args.batch
    t = capi.GGUF_TYPES[args.type]
    host_w = make_layer_weights(args.type)
    layer_bytes = sum(w.nbytes for w in host_w)
    copies = max(2, int(2.5 * L2_BYTES // layer_bytes) + 1)
    layers = [[torch.from_numpy(w).to(dev) for w in host_w] for _ in range(copies)]
    g = torch.Generator().manual_seed(0)
    # four distinct inputs, as in a decoder layer: the attention input (q, k, v), the
    # attention output (o), the MLP input (gate, up) and the gated product (down)
    group = {"q": 0, "k": 0, "v": 0, "o": 1, "gate": 2, "up": 2, "down": 3}
    xin = {}
    for name, _, K in LAYER:
        if group[name] not in xin:
            xin[group[name]] = torch.randn(M, K, generator=g).to(torch.bfloat16).pin_memory()
    x_dev = {k: v.to(dev) for k, v in xin.items()}
    outs = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for _, N, _ in LAYER]
    abytes = algorithmic_bytes(args.type, M)

    def layer_params(weights):
        arr = (capi.GgufMmvqParams * len(LAYER))()
        for i, (W, out, (name, N, K)) in enumerate(zip(weights, outs, LAYER)):
            arr[i] = capi.GgufMmvqParams(M=M, N=N, K=K, A=x_dev[group[name]].data_ptr(), B=W.data_ptr(),
                                         C=out.data_ptr(), type=t, out_dtype=capi.DTYPE_BF16)
        return arr

    layer_args = [layer_params(w) for w in layers]
    ws = torch.empty((max(capi.lib.lsg_gguf_mmvq_batch_workspace_bytes(layer_args[0], len(LAYER)), 256),),
                     dtype=torch.uint8, device=dev)
    # lsg_gguf_mmvq_batch joins consecutive projections of one input into one launch:
    # (q, k, v), o, (gate, up), down -> four mat-vec launches, plus a Q8_1 quantizer launch
    # where the activation is too large to be quantized inside the mat-vec kernel
    # (the library's rule: M * K > 16384)
    joined = []
    for name, _, K in LAYER:
        if not joined or joined[-1][0] != group[name] or joined[-1][2] >= 4:
            joined.append([group[name], K, 0])
        joined[-1][2] += 1
    launches_per_step = sum(1 if M * K <= 16384 else 2 for _, K, _ in joined)

    def layer_step(arr):
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        capi.check(capi.lib.lsg_gguf_mmvq_batch(arr, len(LAYER), ctypes.c_void_p(ws.data_ptr()),
                                                ws.numel(), st))

    # ---- device-resident throughput: one CUDA graph per layer copy ------------------
    for arr in layer_args:
        layer_step(arr)
    torch.cuda.synchronize()
    graphs = []
    for arr in layer_args:
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            layer_step(arr)
        graphs.append(gr)
    for i in range(args.warmup):
        graphs[i % copies].replay()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.15)
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(args.steps):
        graphs[i % copies].replay()
    e1.record()
    torch.cuda.synchronize()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop()
    if world > 1:
        tt = torch.tensor([ms_total], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_total = float(tt.item())
    ms_per_step = ms_total / args.steps
    value = world * abytes / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the operator API, host buffers --------------------------
    e2e_steps = min(args.steps, 400)
    res_host = [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for _, N, _ in LAYER]

    # one prepared batch per layer copy: pointers only; every run() reads the activations
    # from page-locked host memory and writes the results there
    batches = [ops.HostMmvqBatch([(xin[group[name]], W, t, N, K, res)
                                  for W, res, (name, N, K) in zip(weights, res_host, LAYER)])
               for weights in layers]
    for bt in batches:
        bt.capture()

    def e2e_step(i):
        batches[i].run()

    for i in range(10):
        e2e_step(i % copies)
    torch.cuda.synchronize()
    e0.record()
    for i in range(e2e_steps):
        e2e_step(i % copies)
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    if world > 1:
        tt = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_ms = float(tt.item())
    e2e_value = world * abytes / (e2e_ms * 1e-3) / 1e9
    h2d = sum(v.numel() * 2 for v in xin.values())
    d2h = sum(M * N * 2 for _, N, _ in LAYER)

    status = capi.device_status()
    if status != 0:
        raise SystemExit(f"a kernel reported a timed-out device-side wait (code {status})")

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = load_peaks()
    # dominant kernel = the mat-vec; per launch: algorithmic bytes of one projection on
    # average, over the average launch duration (the quantizer launches are inside it).
    n_gemv = len(joined)
    achieved = (abytes / n_gemv) / (ms_per_step * 1e-3 / n_gemv) / 1e9
    line = {
        "metric": f"{args.type.lower()}_mmvq_gbps", "value": value, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic", "config": workload_config(args),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": f"{peak_kind} (copy bandwidth)",
                     "traffic": None, "algorithmic_bytes_per_step": abytes,
                     "launches_per_step": launches_per_step},
        "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "api": "layerstormgemmkernels_b200.ops.HostMmvqBatch.run (lsg_gguf_mmvq_host_batch, captured once into a CUDA graph): the seven projections of a layer, page-locked host tensors in and out"},
        "gpu_launches": args.steps * launches_per_step,
        "clocks": clocks,
    }
    traffic_file = os.path.join(ROOT, "profiles", "traffic.txt")
    if os.path.exists(traffic_file):
        with open(traffic_file) as f:
            for ln in f:
                parts = ln.split()
                if len(parts) == 2 and parts[0] == f"{args.type}_M{M}":
                    line["roofline"]["traffic"] = int(parts[1])
    if not args.no_cpu_baseline and world == 1:
        import oracle
        oracle.build()
        threads = os.cpu_count() or 1
        rng = np.random.default_rng(0)
        xf = {K: rng.standard_normal((M, K)).astype(np.float32) for K in (4096, 14336)}
        cpu_reference_step(args.type, host_w, xf, threads)
        t0 = time.perf_counter()
        n_cpu = 2
        for _ in range(n_cpu):
            cpu_reference_step(args.type, host_w, xf, threads)
        dt = (time.perf_counter() - t0) / n_cpu
        line["cpu_baseline"] = {"value": abytes / dt / 1e9, "unit": "GB/s", "cores": threads,
                                "kind": "port", "ms_per_step": dt * 1e3,
                                "sample": f"{n_cpu} whole-layer steps (7 projections each) after 1 warm-up"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
