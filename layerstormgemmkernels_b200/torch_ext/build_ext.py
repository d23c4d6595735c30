"""Builds the PyTorch extension module `sm120_gemm_kernels` (the reference's module name)
in-tree: <repo>/sm120_gemm_kernels.so, linked against layerstormgemmkernels_b200/liblsg_b200.so.

    python -m layerstormgemmkernels_b200.torch_ext.build_ext
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)


def build(verbose=False):
    from torch.utils.cpp_extension import load
    from .. import build as libbuild
    libbuild.build()
    bdir = os.path.join(HERE, "_build")
    os.makedirs(bdir, exist_ok=True)
    load(name="sm120_gemm_kernels", sources=[os.path.join(HERE, "bindings_python.cpp")],
         extra_include_paths=[os.path.join(ROOT, "include")],
         extra_cflags=["-O2", "-std=c++17"],
         extra_ldflags=[f"-L{PKG}", "-llsg_b200", f"-Wl,-rpath,{PKG}", "-Wl,-rpath,$ORIGIN/layerstormgemmkernels_b200"],
         build_directory=bdir, with_cuda=True, is_python_module=False, verbose=verbose)
    out = os.path.join(ROOT, "sm120_gemm_kernels.so")
    shutil.copyfile(os.path.join(bdir, "sm120_gemm_kernels.so"), out)
    return out


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv))
