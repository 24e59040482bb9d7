"""Stand-ins for the memory checker and race detector that cannot be run on the kernels directly.

* `RedZones`      while active, every tensor the op layer allocates from Python (`torch.empty`, `torch.empty_like`,
                  `torch.zeros`, `Tensor.new_empty`) sits between two guard regions filled with a byte pattern. A kernel
                  that stores outside its output lands in a guard instead of a neighbour's data; `check()` names the
                  allocation whose guard changed. Used around whole forward/backward passes with ragged shapes.
* `repeat_check`  runs a function several times from the same inputs and compares the results bit for bit: a data race
                  between kernels or streams shows up as run-to-run differences. (Kernels that accumulate with
                  floating-point atomics are order-dependent by design and are compared with a tolerance instead.)

The reference has neither; it relies on the eager/compiled PyTorch ops being memory-safe.
"""
from __future__ import annotations

import traceback
from typing import Callable, List

import torch

GUARD_BYTES = 512
PATTERN = 0xA5


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


class RedZones:
    def __init__(self, guard_bytes: int = GUARD_BYTES):
        self.guard_bytes = guard_bytes
        # (byte buffer, offset of the payload, payload bytes, label). The buffers are held until `release()`: a debug run
        # trades memory for the certainty that every guard can still be read when `check()` runs.
        self.records: List[tuple] = []
        self._saved = None

    # ------------------------------------------------------------------ allocation
    def _alloc(self, shape, dtype, device, label):
        dtype = dtype or torch.get_default_dtype()
        item = dtype.itemsize
        nbytes = _numel(shape) * item
        g = self.guard_bytes
        pad = (-nbytes) % 16                                 # the rear guard starts 16-byte aligned like the payload
        raw = self._saved["empty"](g + nbytes + pad + g, dtype=torch.uint8, device=device)
        raw[:g] = PATTERN
        raw[g + nbytes:] = PATTERN
        self.records.append((raw, g, nbytes, label))
        return raw[g:g + nbytes].view(dtype).view(tuple(int(s) for s in shape))

    @staticmethod
    def _label():
        for fr in reversed(traceback.extract_stack(limit=8)):
            if "utils/debug.py" not in fr.filename:
                return f"{fr.filename.rsplit('/', 1)[-1]}:{fr.lineno} ({fr.name})"
        return "?"

    def __enter__(self):
        zones = self
        self._saved = {"empty": torch.empty, "empty_like": torch.empty_like, "zeros": torch.zeros,
                       "new_empty": torch.Tensor.new_empty}

        def _shape_of(args):
            if len(args) == 1 and isinstance(args[0], (tuple, list, torch.Size)):
                return tuple(args[0])
            return tuple(args)

        def empty(*args, dtype=None, device=None, **kw):
            if kw.get("pin_memory") or kw.get("layout") not in (None, torch.strided) or kw.get("memory_format") is not None:
                return zones._saved["empty"](*args, dtype=dtype, device=device, **kw)
            return zones._alloc(_shape_of(args), dtype, device, zones._label())

        def zeros(*args, dtype=None, device=None, **kw):
            if kw:
                return zones._saved["zeros"](*args, dtype=dtype, device=device, **kw)
            return zones._alloc(_shape_of(args), dtype, device, zones._label()).zero_()

        def empty_like(t, dtype=None, device=None, **kw):
            if kw or not t.is_contiguous():
                return zones._saved["empty_like"](t, dtype=dtype, device=device, **kw)
            return zones._alloc(t.shape, dtype or t.dtype, device or t.device, zones._label())

        def new_empty(t, *args, dtype=None, device=None, **kw):
            if kw:
                return zones._saved["new_empty"](t, *args, dtype=dtype, device=device, **kw)
            return zones._alloc(_shape_of(args), dtype or t.dtype, device or t.device, zones._label())

        torch.empty, torch.empty_like, torch.zeros = empty, empty_like, zeros
        torch.Tensor.new_empty = new_empty
        return self

    def __exit__(self, *exc):
        torch.empty, torch.empty_like, torch.zeros = self._saved["empty"], self._saved["empty_like"], self._saved["zeros"]
        torch.Tensor.new_empty = self._saved["new_empty"]
        return False

    # ------------------------------------------------------------------ verification
    def check(self) -> int:
        """Raises naming the first allocation with a damaged guard; returns the number of allocations checked."""
        checked = 0
        for raw, g, nbytes, label in self.records:
            checked += 1
            front, rear = raw[:g], raw[g + nbytes:]
            if not bool((front == PATTERN).all()) or not bool((rear == PATTERN).all()):
                where = "before" if not bool((front == PATTERN).all()) else "after"
                bad = (front if where == "before" else rear) != PATTERN
                first = int(bad.nonzero()[0])
                raise AssertionError(f"red zone {where} the {nbytes}-byte buffer allocated at {label} was overwritten "
                                     f"(first damaged guard byte: {first})")
        return checked

    def release(self):
        self.records.clear()


def repeat_check(fn: Callable[[], object], times: int = 3, atol: float = 0.0):
    """Calls `fn` `times` times and asserts that the tensors it returns (a tensor or a flat tuple/list/dict of
    tensors) are equal across calls: exactly when `atol == 0`, else within `atol` absolute. Returns the first result."""
    def flat(o):
        if isinstance(o, torch.Tensor):
            return [o]
        if isinstance(o, dict):
            return [o[k] for k in sorted(o)]
        return list(o)

    first = None
    for i in range(times):
        cur = [t.detach().clone() for t in flat(fn())]
        if first is None:
            first = cur
            continue
        for j, (a, b) in enumerate(zip(first, cur)):
            if atol == 0.0:
                if not torch.equal(a, b):
                    diff = (a.float() - b.float()).abs().max().item()
                    raise AssertionError(f"run {i} differs from run 0 in output {j} (max abs difference {diff:g})")
            elif not torch.allclose(a.float(), b.float(), rtol=0.0, atol=atol):
                diff = (a.float() - b.float()).abs().max().item()
                raise AssertionError(f"run {i} differs from run 0 in output {j} by {diff:g} > {atol:g}")
    return first


class nvtx_range:
    """`with nvtx_range("name"):` marks a range for timeline tools when SLOWRUN_NVTX=1 and CUDA is present; otherwise it
    does nothing (and costs nothing: the environment is read once)."""
    _on = None

    def __init__(self, name: str):
        if nvtx_range._on is None:
            import os
            nvtx_range._on = os.environ.get("SLOWRUN_NVTX", "0") == "1" and torch.cuda.is_available()
        self.name = name

    def __enter__(self):
        if nvtx_range._on:
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if nvtx_range._on:
            torch.cuda.nvtx.range_pop()
        return False
