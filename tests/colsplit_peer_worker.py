"""Worker of tests/test_gpu_ep_peer.py: one rank of a column-split prefill GEMM whose
all-gather is fused into the GEMM's epilogue (peer-memory stores).  Every rank compares the
gathered [M, N] product with the whole GEMM computed locally (to the last bf16 bit or two:
the two may sum K in a different order)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from layerstormgemmkernels_b200 import capi, distributed as D, ops, quantize as Q  # noqa: E402


def main():
    rank, world, lr = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("nccl", device_id=dev)
    t = capi.Q4_K
    ok = True
    for M, N, K in ((64, 1024, 512), (2304, 512, 1024)):   # fused route, prepared-operand route
        W = Q.quantize_q4_k((np.random.default_rng(7).standard_normal((N, K)) * 0.05).astype(np.float32))
        A = torch.randn(M, K, generator=torch.Generator().manual_seed(11)).to(torch.bfloat16).to(dev)
        n0, n1 = D.column_slab(rank, world, N)
        slab = torch.from_numpy(W[n0:n1]).to(dev)
        full = ops.gguf_mmq(A, torch.from_numpy(W).to(dev), t, N, K)
        cs = D.ColumnSplitPeer(M, N)
        for _ in range(2):   # the output buffer is reused from call to call
            out = cs.gemm(A, slab, t, K)
        torch.cuda.synchronize()
        # the slab and the whole matrix may split K differently (fp32 summation order), so the
        # bf16 results can differ in the last bit
        diff = (out.float() - full.float()).abs().max().item()
        ok = ok and diff <= 2.0 ** -7 * full.float().abs().max().item()
    print(f"COLSPLIT rank {rank} equal={ok} status={capi.device_status()}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
