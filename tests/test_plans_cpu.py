"""Launch plans of the tensor-core kernels, checked on the host for every channel pair they take (no GPU): the
program in ``tests/plans/plan_check.cu`` includes the kernels' own headers, calls ``g3_plan`` / ``w3_plan`` for
2048 shapes and exits with the number of violated invariants (shared memory, stage counts, TMEM columns, the
packing rules of the weight-gradient kernel)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_plans_hold_their_invariants(tmp_path):
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    if not (os.path.exists(nvcc) or shutil.which(nvcc)):
        pytest.skip("nvcc not available")
    exe = str(tmp_path / "plan_check")
    src = os.path.join(ROOT, "tests", "plans", "plan_check.cu")
    build = subprocess.run([nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-o", exe, src],
                           capture_output=True, text=True)
    assert build.returncode == 0, build.stdout + build.stderr
    run = subprocess.run([exe], capture_output=True, text=True)
    assert run.returncode == 0, run.stdout[-2000:]
    assert "2048 shapes" in run.stdout and " 0 violations" in run.stdout
