"""The reference's own GPU test files, unmodified, against the drop-in module.

`__graft_entry__.build()` stages a copy of the reference checkout's tests/ and benchmarks/
under baseline/_ref/ (git-ignored, never part of this repository's history) when the checkout
is present; this test runs those files in a child pytest with the capability shim loaded and
the in-tree `sm120_gemm_kernels.so` first on the path, and requires zero failures.  Without
the staged copy it skips and says so.
"""
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STAGED = os.path.join(ROOT, "baseline", "_ref")
FILES = ["test_gguf_mmvq.py", "test_gguf_grouped_gemm.py", "test_kernels.py"]


def _run(args, timeout):
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([ROOT, os.path.join(ROOT, "tests"), env.get("PYTHONPATH", "")])
    return subprocess.run([sys.executable, *args], cwd=STAGED, env=env, capture_output=True, text=True,
                          timeout=timeout)


@pytest.mark.gpu
@pytest.mark.parametrize("name", FILES)
def test_reference_test_file_passes_unmodified(name):
    path = os.path.join(STAGED, "tests", name)
    if not os.path.exists(path):
        pytest.skip("baseline/_ref/tests is absent: run __graft_entry__.build() where the reference checkout exists")
    if not os.path.exists(os.path.join(ROOT, "sm120_gemm_kernels.so")):
        pytest.fail("sm120_gemm_kernels.so is not built (python -m layerstormgemmkernels_b200.torch_ext.build_ext)")
    r = _run(["-m", "pytest", "-p", "lsg_capshim", "-q", "-x", "--no-header", "-p", "no:cacheprovider",
              os.path.join("tests", name)], timeout=1500)
    tail = (r.stdout + r.stderr)[-3000:]
    summary = re.findall(r"(\d+) (passed|failed|skipped|error)", r.stdout)
    print(f"reference {name}: {summary}")
    counts = {k: int(v) for v, k in summary}
    assert r.returncode == 0, tail
    assert counts.get("passed", 0) > 0 and counts.get("failed", 0) == 0, tail
    # the capability gate must be open: a run that skipped everything proves nothing
    assert counts.get("skipped", 0) < counts.get("passed", 0), tail
