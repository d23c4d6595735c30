"""Worker of tests/test_gpu_ep_peer.py: one rank of a 2-GPU (or N-GPU) expert-parallel MoE
layer.  Runs the layer once with the NCCL all-to-all exchange, three times with the
peer-memory exchange, as two pipelined token halves and as two pipelined expert groups
(each eagerly and from a CUDA graph), and prints
whether the outputs are identical."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from layerstormgemmkernels_b200 import capi, distributed as D, ops, quantize as Q  # noqa: E402


def main():
    rank, world, lr = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("nccl", device_id=dev)
    E, k, H, I, T = 16, 4, 256, 256, 96
    t = capi.Q4_K
    e0, e1 = D.expert_range(rank, world, E)
    g = torch.Generator().manual_seed(3)
    ws = [[Q.quantize_q4_k((torch.randn(n, kk, generator=g) * 0.05).numpy()) for (n, kk) in ((I, H), (I, H), (H, I))]
          for _ in range(E)]
    dw = [[torch.from_numpy(w).to(dev) for w in ws[e]] for e in range(e0, e1)]
    ptr = lambda j: torch.tensor([w[j].data_ptr() for w in dw], dtype=torch.int64, device=dev)  # noqa: E731
    gp, up, dp = ptr(0), ptr(1), ptr(2)
    gg = torch.Generator().manual_seed(1000 + rank)
    hidden = torch.randn(T, H, generator=gg).to(torch.bfloat16).to(dev)
    logits = torch.randn(T, E, generator=gg).to(dev)
    ffn = lambda rows, offs: ops.gguf_moe_ffn(rows, offs, gp, up, dp, t, H, I)  # noqa: E731
    ref = D.ep_moe_layer(hidden, logits, k, E, ffn, ops.moe_route, ops.moe_permutation, ops.moe_permute,
                         ops.moe_unpermute)
    ex = D.EpPeerExchange.make(E, k, H, T, capacity_factor=2.5)
    out = None
    for _ in range(3):   # the buffers are reused from layer to layer
        out = ex.layer(hidden, logits, ffn, ops.moe_route, ops.moe_permutation, ops.moe_unpermute)
    torch.cuda.synchronize()
    print(f"EP_PEER rank {rank} equal={torch.equal(out, ref)} overflow={ex.overflowed()} "
          f"status={capi.device_status()}", flush=True)
    # the same layer as two pipelined halves on side streams, eagerly and replayed from a CUDA graph
    pipe = D.EpPeerPipeline.make(E, k, H, T, chunks=2, capacity_factor=2.5)
    for _ in range(2):
        out2 = pipe.layer(hidden, logits, ffn, ops.moe_route, ops.moe_permutation, ops.moe_unpermute)
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out3 = pipe.layer(hidden, logits, ffn, ops.moe_route, ops.moe_permutation, ops.moe_unpermute)
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    print(f"EP_PIPE rank {rank} equal={torch.equal(out2, ref)} graph_equal={torch.equal(out3, ref)} "
          f"overflow={pipe.overflowed()} status={capi.device_status()}", flush=True)
    # local experts in two groups on side streams (one group's rows travel under the other's GEMMs)
    def ffn_group(rows, offs, lo, hi):
        return ops.gguf_moe_ffn(rows, offs, gp[lo:hi], up[lo:hi], dp[lo:hi], t, H, I)
    grp = D.EpPeerGroups.make(E, k, H, T, groups=2, capacity_factor=2.5)
    for _ in range(2):
        out4 = grp.layer(hidden, logits, ffn_group, ops.moe_route, ops.moe_permutation, ops.moe_unpermute)
    torch.cuda.synchronize()
    dist.barrier()
    graph2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph2):
        out5 = grp.layer(hidden, logits, ffn_group, ops.moe_route, ops.moe_permutation, ops.moe_unpermute)
    for _ in range(2):
        graph2.replay()
    torch.cuda.synchronize()
    print(f"EP_GROUPS rank {rank} equal={torch.equal(out4, ref)} graph_equal={torch.equal(out5, ref)} "
          f"overflow={grp.overflowed()} status={capi.device_status()}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
