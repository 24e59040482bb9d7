"""Host-side replay of the kernels' scheduling arithmetic: `tests/native/sched_model_test.cu` includes the GEMM's own
work iterator, tile mapping and symmetric-mode predicates (csrc/gemm_common.cuh; they compile for the host as well) and
checks, for a thousand shape / worker-count / mode combinations, that every unit of work is covered exactly once. It
stands in for what a memory checker would catch on the device: a tile computed twice, a k-block skipped, a symmetric
element never written."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_gemm_schedule_covers_every_unit_exactly_once(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    exe = str(tmp_path / "sched_model_test")
    src = os.path.join(ROOT, "tests", "native", "sched_model_test.cu")
    build = subprocess.run([nvcc, "-std=c++17", "-O1", "-I", os.path.join(ROOT, "slowrun_b200", "csrc"), "-gencode",
                            "arch=compute_100a,code=sm_100a", "-o", exe, src], capture_output=True, text=True, timeout=600)
    assert build.returncode == 0, build.stderr[-2000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0 and "0 failures" in run.stdout, run.stdout[-3000:]
