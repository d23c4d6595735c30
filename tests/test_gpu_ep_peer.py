"""Expert-parallel MoE layer with the row exchange over peer memory, on two GPUs: identical
output to the NCCL all-to-all exchange.  Skipped on a box with one GPU (the index arithmetic of
the exchange kernels is covered there by test_gpu_moe_routing.py with emulated ranks)."""
import os
import re
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.timeout(300)
def test_peer_exchange_equals_nccl_exchange_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"   # plain peer stores and ring/tree collectives only
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29537", os.path.join(HERE, "ep_peer_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=280)
    # the ranks' lines can arrive glued together on one line of the pipe
    lines = re.findall(r"EP_PEER rank \d+ equal=\w+ overflow=\w+ status=\d+", r.stdout)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert len(lines) == 2, r.stdout[-2000:]
    for ln in lines:
        assert "equal=True" in ln and "overflow=False" in ln and ln.endswith("status=0"), ln
    # the pipelined form (two halves on side streams), eager and graph-replayed
    pipes = re.findall(r"EP_PIPE rank \d+ equal=\w+ graph_equal=\w+ overflow=\w+ status=\d+", r.stdout)
    assert len(pipes) == 2, r.stdout[-2000:] + r.stderr[-2000:]
    for ln in pipes:
        assert " equal=True" in ln and "graph_equal=True" in ln and "overflow=False" in ln and ln.endswith("status=0"), ln
    # local experts in two groups on side streams
    groups = re.findall(r"EP_GROUPS rank \d+ equal=\w+ graph_equal=\w+ overflow=\w+ status=\d+", r.stdout)
    assert len(groups) == 2, r.stdout[-2000:] + r.stderr[-2000:]
    for ln in groups:
        assert " equal=True" in ln and "graph_equal=True" in ln and "overflow=False" in ln and ln.endswith("status=0"), ln


@pytest.mark.timeout(300)
def test_column_split_gemm_with_fused_gather_on_two_gpus():
    """GEMM + all-gather in one kernel: the whole GEMM computed on one GPU, up to summation order."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29538", os.path.join(HERE, "colsplit_peer_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=280)
    lines = re.findall(r"COLSPLIT rank \d+ equal=\w+ status=\d+", r.stdout)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert len(lines) == 2, r.stdout[-2000:]
    for ln in lines:
        assert "equal=True" in ln and ln.endswith("status=0"), ln
