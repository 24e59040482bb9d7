"""Peer-memory collectives: the fused counterpart of `TorchComm` for single-node multi-GPU jobs.

Buffers that other ranks must read (gradient arenas, update chunks, sharded AdamW parameters, flag words) are
allocated through `torch.distributed._symmetric_memory`, which maps every rank's allocation into every other rank's
address space over NVLink. The kernels in `csrc/comm_fused.cu` then read peers directly with plain loads, fused
with the arithmetic that consumes the data (see `ShardedMuonAdamW._step_fused`). NCCL stays available through the
inherited `TorchComm` methods for everything that is not on the hot path (epoch sync, evaluation sums, broadcasts).

The reference has no such layer: all of its gradient traffic is NCCL reduce_scatter / all_gather / all_reduce calls
(train.py:656-760).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib
from .comm import TorchComm

ULL = ctypes.c_ulonglong


class FusedComm(TorchComm):
    name = "fused-p2p"
    fused = True

    def __init__(self, group=None):
        super().__init__(group)
        if not self.active:
            raise RuntimeError("FusedComm needs an initialised multi-rank process group")
        if not torch.cuda.is_available():
            raise RuntimeError("FusedComm needs CUDA")
        import torch.distributed._symmetric_memory as symm
        self._symm = symm
        self._pg = group if group is not None else dist.group.WORLD
        self.device = torch.device("cuda", torch.cuda.current_device())
        self._allocs = []          # (base address, bytes, handle)
        self._guards = []          # (byte buffer, payload bytes, shape, dtype) of every allocation
        self._ptr_cache = {}
        self.epoch = 0
        # How long a device-side barrier waits for each peer before it gives up and reports through the status word.
        # Ranks may legitimately be seconds apart (one of them writes a checkpoint, evaluates, compiles), so the default
        # is generous; tests set it to milliseconds to make a wait run out.
        import os
        self.wait_limit_s = float(os.environ.get("SLOWRUN_PEER_WAIT_S", "60"))
        self.flags = self.alloc((64,), torch.int32)
        self.flag_ptrs = self.peer_ptrs(self.flags)
        self.progress = self.alloc((64,), torch.int32)      # per-rank progress counters (signal / wait_for)
        self.progress_ptrs = self.peer_ptrs(self.progress)
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    # ------------------------------------------------------------------ symmetric allocation
    GUARD_BYTES = 256
    GUARD_PATTERN = 0x5A

    def alloc(self, shape, dtype) -> torch.Tensor:
        """Zero-filled tensor mapped by every rank (collective call: all ranks must allocate in the same order). Every
        allocation ends in a guard region filled with a byte pattern: peers write into these buffers with plain and
        multicast stores, and a store that ran past the end of a buffer would otherwise land in whatever the allocator put
        next. `check_guards()` verifies them."""
        n = 1
        for d in shape:
            n *= int(d)
        item = torch.empty((), dtype=dtype).element_size()
        payload = (n * item + 15) // 16 * 16
        raw = self._symm.empty((payload + self.GUARD_BYTES,), dtype=torch.uint8, device=self.device)
        raw.zero_()
        raw[payload:] = self.GUARD_PATTERN
        hdl = self._symm.rendezvous(raw, self._pg)
        self._allocs.append((raw.data_ptr(), payload + self.GUARD_BYTES, hdl))
        self._guards.append((raw, payload, tuple(int(d) for d in shape), dtype))
        return raw[:n * item].view(dtype).view(tuple(int(d) for d in shape))

    def check_guards(self) -> int:
        """Synchronising check of the guard region behind every symmetric allocation of this rank; raises naming the
        buffer whose guard was overwritten. Returns the number of buffers checked."""
        for raw, payload, shape, dtype in self._guards:
            g = raw[payload:]
            if not bool((g == self.GUARD_PATTERN).all()):
                first = int((g != self.GUARD_PATTERN).nonzero()[0])
                raise AssertionError(f"rank {self.rank}: guard behind the symmetric buffer {shape} {dtype} was overwritten "
                                     f"(first damaged byte at +{first})")
        return len(self._guards)

    def peer_ptrs(self, t: torch.Tensor):
        """ctypes array with the address of `t` (or of a view into an allocated tensor) on every rank."""
        key = (t.data_ptr(), t.numel())
        arr = self._ptr_cache.get(key)
        if arr is not None:
            return arr
        a = t.data_ptr()
        for base, nbytes, hdl in self._allocs:
            if base <= a < base + max(nbytes, 1):
                ptrs = list(hdl.buffer_ptrs)
                mine = ptrs[hdl.rank]
                off = a - mine
                if off < 0:
                    raise RuntimeError("symmetric allocation does not start at the handle's buffer pointer")
                arr = (ULL * self.world)(*[int(p) + off for p in ptrs])
                self._ptr_cache[key] = arr
                return arr
        raise KeyError("tensor was not allocated through FusedComm.alloc")

    # ------------------------------------------------------------------ device-side barrier
    def multicast_ptr(self, t: torch.Tensor) -> int:
        """NVLS multicast address of `t` (reads through it return the sum over all ranks, reduced in the switch), or 0
        when the allocation has no multicast mapping or SLOWRUN_MULTIMEM=0."""
        import os
        if os.environ.get("SLOWRUN_MULTIMEM", "1") == "0":
            return 0
        a = t.data_ptr()
        for base, nbytes, hdl in self._allocs:
            if base <= a < base + max(nbytes, 1):
                try:
                    mc = int(hdl.multicast_ptr or 0)
                except Exception:  # noqa: BLE001
                    mc = 0
                if mc == 0:
                    return 0
                return mc + (a - int(list(hdl.buffer_ptrs)[hdl.rank]))
        return 0

    def device_barrier(self):
        """All ranks' preceding work on the current stream is complete and visible before any rank proceeds."""
        self.epoch += 1
        rc = _lib.fn("sr_peer_barrier", [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_uint, ctypes.c_void_p,
                                         ctypes.c_ulonglong, ctypes.c_void_p])(
            ctypes.cast(self.flag_ptrs, ctypes.c_void_p), self.rank, self.world, self.epoch,
            _lib.status_buffer(self.device).data_ptr(), int(self.wait_limit_s * 1e9), _lib.stream_ptr())
        _lib.check_rc(rc, "sr_peer_barrier")

    def signal(self, value: int):
        """Publish on the current stream: everything this rank enqueued before is done; its counter becomes `value`
        (values must grow monotonically over the run)."""
        rc = _lib.fn("sr_peer_signal", [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_uint, ctypes.c_void_p])(
            ctypes.cast(self.progress_ptrs, ctypes.c_void_p), self.rank, self.world, int(value) & 0xFFFFFFFF, _lib.stream_ptr())
        _lib.check_rc(rc, "sr_peer_signal")

    def wait_for(self, value: int):
        """Hold the current stream until every rank's counter has reached `value` (bounded; a wait that runs out sets
        the status word and the kernels that follow skip their work)."""
        rc = _lib.fn("sr_peer_wait", [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_uint, ctypes.c_void_p,
                                      ctypes.c_ulonglong, ctypes.c_void_p])(
            ctypes.cast(self.progress_ptrs, ctypes.c_void_p), self.rank, self.world, int(value) & 0xFFFFFFFF,
            _lib.status_buffer(self.device).data_ptr(), int(self.wait_limit_s * 1e9), _lib.stream_ptr())
        _lib.check_rc(rc, "sr_peer_wait")

    # ------------------------------------------------------------------ fused primitives
    def reduce_from_peers(self, src: torch.Tensor, offset: int, out: torch.Tensor):
        """out[i] = sum_r src_r[offset + i], fp32 result; src is a symmetric fp32 or bf16 tensor."""
        rc = _lib.fn("sr_reduce_multi", [ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_void_p, ctypes.c_long, ctypes.c_int,
                                         ctypes.c_void_p, ctypes.c_void_p])(
            ctypes.cast(self.peer_ptrs(src), ctypes.c_void_p), self.world, offset, out.data_ptr(), out.numel(),
            int(src.dtype == torch.bfloat16), _lib.status_buffer(self.device).data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "sr_reduce_multi")

    def gather_slices(self, buf: torch.Tensor):
        """Every rank owns slice `rank` of `buf` along dim 0; pull the other ranks' slices from their replicas."""
        slice_bytes = buf.numel() * buf.element_size() // self.world
        rc = _lib.fn("sr_gather_multi", [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_long, ctypes.c_void_p, ctypes.c_void_p])(
            ctypes.cast(self.peer_ptrs(buf), ctypes.c_void_p), self.world, self.rank, slice_bytes,
            _lib.status_buffer(self.device).data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "sr_gather_multi")
