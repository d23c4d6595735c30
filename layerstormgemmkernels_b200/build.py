"""Builds the C-ABI shared library (liblsg_b200.so) for sm_100a with nvcc.

Usage: python -m layerstormgemmkernels_b200.build [--force] [--verbose]

Objects are compiled in parallel into csrc/_obj and linked into
layerstormgemmkernels_b200/liblsg_b200.so.  nvcc cross-compiles, so no GPU is needed to build.
"""
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(HERE, "liblsg_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

# (source, object suffix, extra flags)
def _units():
    units = []
    for name in sorted(os.listdir(CSRC)):
        if not name.endswith(".cu"):
            continue
        if name == "mmvq_inst.cu":
            for t in range(8):
                units.append((name, f"mmvq_inst_t{t}.o", [f"-DLSG_MMVQ_TYPE={t}"]))
        else:
            units.append((name, name[:-3] + ".o", []))
    return units


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _digest(extra):
    h = hashlib.sha256()
    for root in (CSRC, os.path.join(os.path.dirname(HERE), "include")):
        for name in sorted(os.listdir(root)):
            if name.endswith((".cu", ".cuh", ".h")):
                with open(os.path.join(root, name), "rb") as f:
                    h.update(name.encode())
                    h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + extra).encode())
    return h.hexdigest()


def build(force=False, verbose=False, extra_flags=()):
    """Compiles every CUDA source for sm_100a and links the shared library.  Returns its path."""
    extra = list(extra_flags)
    stamp = os.path.join(OBJ, "stamp")
    digest = _digest(extra)
    if not force and os.path.exists(LIB) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return LIB
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()

    def compile_one(unit):
        src, obj, flags = unit
        cmd = [nvcc, *NVCC_FLAGS, *extra, *flags, "-c", os.path.join(CSRC, src), "-o",
               os.path.join(OBJ, obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return unit, r

    units = _units()
    with cf.ThreadPoolExecutor(max_workers=min(len(units), os.cpu_count() or 4)) as ex:
        results = list(ex.map(compile_one, units))
    for (src, obj, _), r in results:
        if verbose and (r.stdout or r.stderr):
            sys.stderr.write(f"--- {obj}\n{r.stdout}{r.stderr}")
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src} ({obj}):\n{r.stdout}\n{r.stderr}")
    objs = [os.path.join(OBJ, obj) for _, obj, _ in units]
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs,
            "-lcudart"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    with open(stamp, "w") as f:
        f.write(digest)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv,
                 extra_flags=["-Xptxas", "-v"] if "--ptxas" in sys.argv else [])
    print(path)
