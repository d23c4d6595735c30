"""pytest plugin: makes torch report compute capability (12, 0).

The reference's GPU tests and benchmarks skip themselves unless
torch.cuda.get_device_capability()[0] >= 12 (tests/test_gguf_mmvq.py:34-41,
tests/test_gguf_grouped_gemm.py:37-44, tests/test_kernels.py:36-40 of
kkontosis/LayerStoRmGemmKernels): a gate on the GPU their kernels were written for, not on
anything the operators' contract needs.  Loading this plugin (`pytest -p lsg_capshim`, with
this directory on PYTHONPATH) before collection lets those files run unmodified against the
drop-in module `sm120_gemm_kernels` on a B200.  Importing it as a plain module has the same
effect (`python -c "import lsg_capshim; ..."`, used for the reference's benchmark scripts).
"""
import torch

_real = torch.cuda.get_device_capability


def _capability(device=None):
    major, minor = _real(device)
    return (12, 0) if major >= 10 else (major, minor)


torch.cuda.get_device_capability = _capability
