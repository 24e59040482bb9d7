"""Checkpoints.

* Weight snapshots in the reference's layout: a flat `{parameter name: fp32 CPU tensor}` dict over
  `named_parameters()` (train.py:1231-1243), loadable by the reference's `load_state_dict_into_model`
  (train.py:182-186) and vice versa. Ring buffer of the last N, recency-weighted weight averaging
  (tiny/train.py:1573-1593), zero-initialised bias-corrected weight EMA (tiny/train.py:1336-1337, 1448-1449, 1541-1549).
* A full-state checkpoint (weights + sharded optimizer state per rank + RNG + loader position + step) for true
  resume in every track; the reference only has that for the unlimited track (unlimited/train.py:1897-1918).
"""
from __future__ import annotations

import os
from typing import Dict, List

import torch


def named_param_snapshot(model) -> Dict[str, torch.Tensor]:
    return {name: p.data.float().cpu() for name, p in model.named_parameters()}


@torch.no_grad()
def load_named_params(model, state: Dict[str, torch.Tensor]):
    for name, p in model.named_parameters():
        if name in state:
            p.data.copy_(state[name].to(p.device, dtype=p.dtype))
    if getattr(model, "arena", None) is not None:
        model.arena.refresh_shadows()


class CheckpointRing:
    """Keeps the last `keep` epoch snapshots on disk (rank 0 writes; every rank tracks the paths)."""

    def __init__(self, directory: str, keep: int, is_master: bool):
        self.dir, self.keep, self.is_master = directory, keep, is_master
        self.paths: List[str] = []
        if keep > 0 and is_master:
            os.makedirs(directory, exist_ok=True)

    def save(self, model, epoch: int) -> str:
        path = os.path.join(self.dir, f"epoch_{epoch:03d}.pt")
        if self.is_master:
            torch.save(named_param_snapshot(model), path)
        self.paths.append(path)
        if len(self.paths) > self.keep:
            old = self.paths.pop(0)
            if self.is_master and os.path.exists(old):
                os.remove(old)
        return path


def recency_weights(n: int, mode: str = "weighted"):
    if mode == "equal":
        return [1.0 / n] * n
    raw = list(range(1, n + 1))
    return [w / sum(raw) for w in raw]


@torch.no_grad()
def average_checkpoints_into(model, paths: List[str], weights, comm=None, is_master=True):
    """Recency-weighted weight average of saved snapshots, computed on rank 0 and broadcast (tiny/train.py:1573-1587)."""
    if comm is not None:
        comm.barrier()
    if is_master:
        cks = [torch.load(p, map_location="cpu", weights_only=True) for p in paths]
        merged = {name: sum(weights[i] * cks[i][name].float() for i in range(len(cks))) for name in cks[0]}
        for name, p in model.named_parameters():
            if name in merged:
                p.data.copy_(merged[name].to(p.device, p.dtype))
    if comm is not None:
        comm.barrier()
        for p in model.parameters():
            comm.broadcast(p.data, src=0)
    if getattr(model, "arena", None) is not None:
        model.arena.refresh_shadows()


class WeightEMA:
    """ema <- lerp(ema, p, 1-beta) every `every` steps, zero-initialised; `copy_into` applies the bias correction."""

    def __init__(self, model, decay_per_epoch: float, every: int, steps_per_epoch: float):
        self.every = every
        self.beta = decay_per_epoch ** (every / steps_per_epoch) if every > 0 else 0.0
        self.params = list(model.parameters())
        self.ema = [torch.zeros_like(p) for p in self.params] if every > 0 else None
        self.updates = 0

    @torch.no_grad()
    def maybe_update(self, step: int):
        if self.ema is not None and step % self.every == 0:
            torch._foreach_lerp_(self.ema, [p.data for p in self.params], 1 - self.beta)
            self.updates += 1

    @torch.no_grad()
    def copy_into(self, model):
        if self.ema is None or self.updates == 0:
            return False
        corr = 1.0 / (1.0 - self.beta ** self.updates)
        for p, e in zip(self.params, self.ema):
            p.data.copy_(e * corr)
        if getattr(model, "arena", None) is not None:
            model.arena.refresh_shadows()
        return True


def save_full_state(path: str, model, optimizer, loader_state, step: int, extra=None, rank: int = 0, world_size: int = 1):
    """Per-rank resume file `<path>.rank<r>`: weights (rank 0 only), this rank's optimizer shard, RNG states (torch CPU and
    CUDA generators, the dropout kernels' call-site salt and device step counter), the loader position
    (`TokenLoader.state()`), and whatever the trainer passes in `extra`. Written to a temporary name and renamed, so a run
    killed while saving leaves the previous file intact."""
    from ..ops import functional as ops
    state = {
        "step": step,
        "world_size": world_size,
        "optimizer": optimizer.state_dict(),
        "rng_cpu": torch.get_rng_state(),
        "rng_cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None,
        "dropout": ops.dropout_rng_state(),
        "loader": loader_state,
        "extra": extra or {},
    }
    if rank == 0:
        state["model"] = named_param_snapshot(model)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = f"{path}.rank{rank}.tmp"
    torch.save(state, tmp)
    os.replace(tmp, f"{path}.rank{rank}")


def full_state_exists(path: str, rank: int = 0) -> bool:
    return bool(path) and os.path.exists(f"{path}.rank{rank}") and os.path.exists(f"{path}.rank0")


def load_full_state(path: str, model, optimizer, rank: int = 0, world_size: int = 1):
    from ..ops import functional as ops
    state = torch.load(f"{path}.rank{rank}", map_location="cpu", weights_only=False)
    if state.get("world_size", world_size) != world_size:
        raise RuntimeError(f"resume file was written by {state['world_size']} ranks, this run has {world_size}: the "
                           "optimizer state is sharded by rank and cannot be re-dealt")
    if rank == 0:
        weights = state["model"]
    else:
        weights = torch.load(f"{path}.rank0", map_location="cpu", weights_only=False)["model"]
    load_named_params(model, weights)
    optimizer.load_state_dict(state["optimizer"])
    torch.set_rng_state(state["rng_cpu"])
    if state.get("rng_cuda") is not None and torch.cuda.is_available():
        torch.cuda.set_rng_state(state["rng_cuda"])
    if state.get("dropout") is not None:
        ops.set_dropout_rng_state(state["dropout"])
    return state
