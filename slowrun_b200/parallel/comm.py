"""Process-group bootstrap and the collective layer the optimizer talks to.

`init_distributed()` reads the torchrun environment (RANK / LOCAL_RANK / WORLD_SIZE), creates an NCCL group on GPUs
or a Gloo group on CPU, and returns a `DistInfo`. Without those variables the job is single-process and every
collective below degenerates to a no-op — the reference requires torchrun even for one GPU because its optimizer
calls dist.get_rank() unconditionally (train.py:146-149, 748, 948-957).

`TorchComm` is the library path (NCCL / Gloo through torch.distributed): the measured baseline and the fallback.
Gradients are reduced with SUM and the 1/world factor is folded into the consuming kernel, because Gloo has no AVG
(the reference uses ReduceOp.AVG, train.py:661-682). `slowrun_b200.parallel.fused` provides the same interface on
top of peer-memory kernels.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class DistInfo:
    distributed: bool
    rank: int
    local_rank: int
    world_size: int
    device: torch.device


def get_dist_info():
    if all(k in os.environ for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE")):
        return True, int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    return False, 0, 0, 1


def init_distributed(device: Optional[str] = None, timeout_s: Optional[float] = None) -> DistInfo:
    ddp, rank, local_rank, world = get_dist_info()
    use_cuda = torch.cuda.is_available() and device != "cpu"
    if use_cuda:
        dev = torch.device("cuda", local_rank if ddp else 0)
        torch.cuda.set_device(dev)
    else:
        dev = torch.device("cpu")
    if ddp and not dist.is_initialized():
        kw = {}
        if timeout_s is not None:
            kw["timeout"] = datetime.timedelta(seconds=timeout_s)
        if use_cuda:
            dist.init_process_group(backend="nccl", device_id=dev, **kw)
        else:
            dist.init_process_group(backend="gloo", **kw)
        dist.barrier()
    return DistInfo(ddp, rank, local_rank, world, dev)


def shutdown():
    if dist.is_initialized():
        dist.destroy_process_group()


def print0(*a, **kw):
    if int(os.environ.get("RANK", 0)) == 0:
        print(*a, **kw)


class _Done:
    def wait(self):
        return None


class TorchComm:
    """Collectives through torch.distributed; all of them are no-ops in a single-process job."""

    name = "torch"

    def __init__(self, group=None):
        self.group = group
        self.active = dist.is_initialized() and dist.get_world_size(group) > 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1

    def reduce_scatter_sum(self, out, inp, async_op=True):
        """out[chunk...] = sum over ranks of inp[rank*chunk:(rank+1)*chunk] along dim 0."""
        if not self.active:
            out.copy_(inp[: out.shape[0]])
            return _Done()
        w = dist.reduce_scatter_tensor(out, inp, op=dist.ReduceOp.SUM, group=self.group, async_op=async_op)
        return w if async_op else _Done()

    def all_gather(self, out, inp, async_op=True):
        if not self.active:
            out[: inp.shape[0]].copy_(inp)
            return _Done()
        w = dist.all_gather_into_tensor(out, inp, group=self.group, async_op=async_op)
        return w if async_op else _Done()

    def all_reduce_sum(self, t, async_op=True):
        if not self.active:
            return _Done()
        w = dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group, async_op=async_op)
        return w if async_op else _Done()

    def all_reduce_max(self, t):
        if self.active:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return t

    def broadcast(self, t, src=0):
        """`src` counts inside this communicator's group (rank 0 of a node group is that node's first rank)."""
        if self.active:
            if self.group is None:
                dist.broadcast(t, src=src)
            else:
                dist.broadcast(t, group=self.group, group_src=src)
        return t

    def barrier(self):
        if self.active:
            dist.barrier(group=self.group)
