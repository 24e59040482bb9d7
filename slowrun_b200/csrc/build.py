"""Builds the sm_100a kernel library in-tree with nvcc.

All kernels are plain CUDA with `extern "C"` launchers (raw pointers + stream), so no torch headers are needed and
a full rebuild takes seconds. The result is `slowrun_b200/_kernels.so`, loaded through ctypes by
`slowrun_b200.ops._lib`. The reference has no build step: its only native kernel is NVRTC-compiled at import
(tiny/cuda_kernels.py:305-312).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

CSRC = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(CSRC)
# SLOWRUN_DEBUG_CHECKS=1 selects a second library built with -DSR_DEBUG_CHECKS (index and alignment checks inside the
# kernels that report through the status word; see SR_DEBUG_CHECK in sm100_common.cuh). Both can sit side by side.
DEBUG_CHECKS = os.environ.get("SLOWRUN_DEBUG_CHECKS", "0") == "1"
OUT = os.path.join(PKG, "_kernels_debug.so" if DEBUG_CHECKS else "_kernels.so")
OBJ_DIR = os.path.join(CSRC, "build_debug" if DEBUG_CHECKS else "build")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
] + (["-DSR_DEBUG_CHECKS"] if DEBUG_CHECKS else [])


def sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; cannot build slowrun_b200 kernels")
    return nvcc


def _digest() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(f.encode())
                h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    stamp = OUT + ".sha"
    if not (os.path.exists(OUT) and os.path.exists(stamp)):
        return False
    with open(stamp) as fh:
        return fh.read().strip() == _digest()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu file for sm_100a and link `_kernels.so`. Returns the library path."""
    if not force and is_current():
        return OUT
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)

    def compile_one(src: str) -> tuple[str, str]:
        obj = os.path.join(OBJ_DIR, src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
        return obj, res.stderr

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        results = list(ex.map(compile_one, sources()))
    objs = [o for o, _ in results]
    with open(os.path.join(OBJ_DIR, "ptxas.log"), "w") as fh:
        for _, log in results:
            fh.write(log)
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    cmd = [nvcc, "-shared", "-o", OUT, *objs, "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    with open(OUT + ".sha", "w") as fh:
        fh.write(_digest())
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
