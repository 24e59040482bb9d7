"""ctypes loader for the in-tree sm_100a kernel library (`slowrun_b200/_kernels.so`).

The kernels are launched through `extern "C"` entry points that take raw device pointers and a CUDA stream, so
no torch C++ extension is involved. On a machine with a GPU the library is mandatory: ops raise if it is missing
rather than silently running a PyTorch fallback.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# SLOWRUN_DEBUG_CHECKS=1 loads the library variant built with the in-kernel index/alignment checks (csrc/build.py)
_SO = os.path.join(_PKG, "_kernels_debug.so" if os.environ.get("SLOWRUN_DEBUG_CHECKS", "0") == "1" else "_kernels.so")
_lock = threading.Lock()
_lib = None
_status = {}

c_void_p, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


class KernelStatusError(RuntimeError):
    """A kernel abandoned a bounded wait and reported it through its status word."""


def library_path() -> str:
    return _SO


def available() -> bool:
    """True when CUDA kernels can run here (a GPU is present)."""
    return torch.cuda.is_available()


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(_SO):
                from ..csrc import build as _build
                _build.build()
            _lib = ctypes.CDLL(_SO)
            if torch.cuda.is_available():
                # resolve the driver's tensor-map encoder here, on the loading thread, for every later caller
                # (backward passes call the GEMMs from autograd's worker thread)
                _lib.sr_runtime_init.restype = ctypes.c_int
                if _lib.sr_runtime_init() != 0:
                    raise RuntimeError("the CUDA driver does not export cuTensorMapEncodeTiled; the sm_100a kernels cannot run")
            if os.environ.get("SR_GEMM_PAIR", "1") == "0":
                _lib.sr_gemm_set_pair_mode(0)
    return _lib


_fn_cache = {}
launch_count = 0     # launcher calls made so far (each launcher enqueues one or more kernels)


def fn(name: str, argtypes, restype=c_int):
    """Returns a callable for the `extern "C"` launcher `name`; every call through it is counted."""
    w = _fn_cache.get(name)
    if w is not None:
        return w
    f = getattr(lib(), name)
    f.argtypes = argtypes
    f.restype = restype

    def call(*args, _f=f):
        global launch_count
        launch_count += 1
        return _f(*args)

    _fn_cache[name] = call
    return call


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def status_buffer(device=None) -> torch.Tensor:
    """int32[4] device buffer shared by every kernel launched from this process on `device`."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    buf = _status.get(key)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=dev)
        _status[key] = buf
    return buf


def check_status(device=None, reset: bool = True) -> None:
    """Synchronising check of the status word; raises KernelStatusError if any kernel gave up a wait."""
    buf = status_buffer(device)
    vals = buf.tolist()
    if vals[0] != 0:
        if reset:
            buf.zero_()
        raise KernelStatusError(
            f"kernel status: code={vals[0]} site={vals[1]} block={vals[2]} detail={vals[3]} "
            "(1 = mbarrier wait ran out, 2 = peer wait ran out, 3 = bad argument, 4 = debug-build check failed)")


def check_rc(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what}: launcher returned {rc}")
