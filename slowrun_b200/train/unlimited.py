"""Unlimited track: chains of cyclic-LR snapshots per node, chain distillation, weight perturbation, per-snapshot
p(ground-truth) caches on a held-out fitness slice, gradient-based ensemble selection and ensemble evaluation,
with cycle-boundary resume.

Behaviour follows the reference's unlimited trainer (unlimited/train.py:1001-1306 ensemble machinery, 1312-1941
snapshot run, 1947-2234 main): each node trains `num_models / n_nodes` snapshots one after the other ("cycles" of
`epochs_per_cycle` epochs), LR falls linearly from 1 to `lr_floor` inside a cycle, WD moves against the LR, the
batch is `bs_floor` in the outer quarters of the cycle list and the full batch in the middle, gradients are
data-parallel over the node's GPUs with a global-norm clip at 1.0 and an un-sharded optimizer on every rank (the
reference wraps the model in DistributedDataParallel, unlimited/train.py:1400); from `distill_after_cycles` on the
loss is (1-a)(CE + mtp) + a T^2 KL(student/T || teacher/T) against the previous snapshot.
"""
from __future__ import annotations

import json
import math
import os
import time
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

import copy
import dataclasses

from ..config import TrainConfig
from ..data.loader import EnsembleTokenLoader, TokenLoader
from ..models.gpt import build_model
from ..optim.groups import build_param_groups
from ..optim.muon_adamw import ShardedMuonAdamW
from ..parallel.comm import DistInfo, TorchComm, init_distributed, print0
from .checkpoint import load_named_params
from .evaluate import default_token_bytes, evaluate_bpb
from .selection import select_members


# Per-node hyper-parameter overrides for ensemble diversity, keyed by node rank (unlimited/train.py:62-68, 1325-1330,
# 2046). Any field of TrainConfig may be overridden (the reference uses lr_multiplier, weight_decay, label_smoothing,
# lr_floor, warmup_frac, warmdown_frac and documents distill_alpha / distill_temperature). Filled from the
# `node_overrides` argument of UnlimitedTrainer or from the JSON in $SLOWRUN_NODE_OVERRIDES; empty = every node alike.
NODE_OVERRIDES: Dict[int, dict] = {}


def config_for_node(cfg: TrainConfig, node_rank: int, overrides: Optional[Dict[int, dict]] = None) -> TrainConfig:
    """Copy of `cfg` with this node's overrides applied; unknown keys are an error."""
    table = dict(NODE_OVERRIDES)
    env = os.environ.get("SLOWRUN_NODE_OVERRIDES")
    if env:
        table.update({int(k): v for k, v in json.loads(env).items()})
    if overrides:
        table.update({int(k): v for k, v in overrides.items()})
    mine = table.get(node_rank, {})
    out = copy.deepcopy(cfg)
    alias = {"warmup_frac": "warmup_ratio", "warmdown_frac": "cycle_warmdown_frac"}
    fields = {f.name for f in dataclasses.fields(out)}
    for k, v in mine.items():
        k = alias.get(k, k)
        if k == "label_smoothing":
            out.model.label_smoothing = v
        elif k == "cycle_warmdown_frac":
            out.cycle_warmdown_frac = v
        elif k in fields:
            setattr(out, k, v)
        else:
            raise KeyError(f"node override {k!r} is not a training option")
    out.node_overrides = {str(k): v for k, v in table.items()}
    return out


class LayerBuckets:
    """Gradient buffers grouped by the layer that writes them, as slices of the stacked arenas: the unit of the
    reductions that run while the backward pass is still going (the reference gets this from DistributedDataParallel's
    25 MB buckets, unlimited/train.py:1400, 1627-1630)."""

    def __init__(self, model):
        a = model.arena
        owner = {}
        for i, blk in enumerate(model.transformer.h):
            for p in blk.parameters():
                owner[id(p)] = i
        for k, lin in model.ve_projs.items():
            owner[id(lin.weight)] = int(k)
        self.n_layer = len(model.transformer.h)
        if model.mtp_weight > 0:
            for p in list(model.mtp_block.parameters()) + list(model.mtp_proj.parameters()):
                owner[id(p)] = self.n_layer
        self.per_layer: Dict[int, List[torch.Tensor]] = {}
        rest: List[torch.Tensor] = []
        for g in a.groups.values():
            start = 0
            for s in range(1, g.n + 1):
                if s == g.n or owner.get(id(g.params[s])) != owner.get(id(g.params[start])):
                    L = owner.get(id(g.params[start]))
                    (rest if L is None else self.per_layer.setdefault(L, [])).append(g.G[start:s])
                    start = s
        rest.append(a.head_grad)
        if a.small_grads.numel():
            rest.append(a.small_grads)
        rest += [p.grad for p in a.other_params]
        self.rest = rest

    def all_buffers(self):
        return [b for bs in self.per_layer.values() for b in bs] + self.rest


class OverlappedAllReduce:
    """Data-parallel gradient averaging that starts during the backward pass of the last micro-batch: when the
    backward has moved past layer i, the buffers of layer i + 1 are final and their all-reduce is issued; what is left
    (first layer, embeddings, head, small parameters) follows after the pass. One reduction per arena slice, not per
    tensor."""

    def __init__(self, model, comm: TorchComm):
        self.model, self.comm = model, comm
        self.buckets = LayerBuckets(model)
        self.handles, self.launched = [], set()

    def _launch(self, L):
        if L in self.launched or L not in self.buckets.per_layer:
            return
        self.launched.add(L)
        for b in self.buckets.per_layer[L]:
            self.handles.append(self.comm.all_reduce_sum(b))

    def arm(self):
        self.handles, self.launched = [], set()
        top = self.buckets.n_layer

        def hook(i):
            # layers are visited from the last to the first; everything above i has finished
            for L in range(top, i, -1):
                self._launch(L)
        self.model.layer_done_hook = hook

    def finish(self):
        self.model.layer_done_hook = None
        for L in sorted(self.buckets.per_layer, reverse=True):
            self._launch(L)
        self.handles += [self.comm.all_reduce_sum(b) for b in self.buckets.rest]
        for h in self.handles:
            h.wait()
        inv = 1.0 / self.comm.world
        for b in self.buckets.all_buffers():
            b.mul_(inv)
        self.handles = []


class _Single(TorchComm):
    """Optimizer-side communicator of a replicated (non-sharded) optimizer: every collective is a no-op."""

    def __init__(self):
        self.group, self.active, self.rank, self.world = None, False, 0, 1


class CyclePlan:
    """Per-cycle batch size, length and LR / WD multipliers (unlimited/train.py:1446-1494)."""

    def __init__(self, cfg: TrainConfig, num_cycles: int, tokens_per_epoch: int, tokens_per_fwdbwd_node: int):
        self.cfg = cfg
        peak, floor = cfg.total_batch_size, cfg.bs_floor
        assert peak % tokens_per_fwdbwd_node == 0 and floor % tokens_per_fwdbwd_node == 0 and 0 < floor <= peak
        tokens_per_cycle = tokens_per_epoch * cfg.epochs_per_cycle

        def bs(c):
            if cfg.bs_schedule == "flat" or num_cycles == 1:
                return peak
            amp = 1.0 - abs(2.0 * c / (num_cycles - 1) - 1.0)
            return peak if amp >= 0.5 else floor
        self.batch_sizes = [bs(c) for c in range(num_cycles)]
        self.lengths = [max(1, round(tokens_per_cycle / b)) for b in self.batch_sizes]
        self.grad_accums = [b // tokens_per_fwdbwd_node for b in self.batch_sizes]
        self.total_iterations = sum(self.lengths)
        self.warmup_frac, self.warmdown_frac = cfg.warmup_ratio, float(getattr(cfg, "cycle_warmdown_frac", 0.0))

    def signature(self):
        return {"batch_sizes": self.batch_sizes, "lengths": self.lengths}

    def lr_multiplier(self, step_in_cycle: int, cycle_length: int) -> float:
        f = self.cfg.lr_floor
        wu = int(cycle_length * self.warmup_frac)
        wd = int(cycle_length * self.warmdown_frac)
        decay = cycle_length - wu - wd
        if step_in_cycle < wu:
            return f + (1.0 - f) * step_in_cycle / wu
        if step_in_cycle < wu + decay:
            return f + (1.0 - f) * (1.0 - (step_in_cycle - wu) / decay)
        return f * 0.5 * (1.0 + math.cos(math.pi * (step_in_cycle - wu - decay) / wd))

    def wd_multiplier(self, step_in_cycle: int, cycle_length: int) -> float:
        span = 1.0 - self.cfg.lr_floor
        if self.cfg.wd_schedule == "flat" or span <= 0:
            return 1.0
        progress = (1.0 - self.lr_multiplier(step_in_cycle, cycle_length)) / span
        return self.cfg.wd_floor + (1.0 - self.cfg.wd_floor) * progress


def perturb_scale(cfg: TrainConfig, cycle: int, num_cycles: int) -> float:
    """Cosine decay of the perturbation scale from perturb_scale to perturb_scale_min over the chain."""
    if num_cycles <= 1:
        return cfg.perturb_scale
    t = cycle / (num_cycles - 1)
    return cfg.perturb_scale_min + 0.5 * (cfg.perturb_scale - cfg.perturb_scale_min) * (1 + math.cos(math.pi * t))


@torch.no_grad()
def perturb_weights(model, scale: float, seed: int, comm: Optional[TorchComm]):
    """p += N(0, (scale * std(p))^2), generated on the CPU from `seed` and made identical on all ranks by broadcast
    (unlimited/train.py:1292-1306, 1884-1895)."""
    g = torch.Generator().manual_seed(seed)
    for p in model.parameters():
        if p.numel() < 2:
            continue
        noise = torch.randn(p.shape, generator=g, dtype=torch.float32) * (scale * float(p.data.float().std()))
        p.data.add_(noise.to(p.device, p.dtype))
    if comm is not None and comm.active:
        for p in model.parameters():
            comm.broadcast(p.data, src=0)
    if getattr(model, "arena", None) is not None:
        model.arena.refresh_shadows()


def allreduce_gradients(model, comm: TorchComm):
    """Data-parallel gradient averaging over the arenas (a handful of large buffers instead of one call per tensor)."""
    if not comm.active:
        return
    a = model.arena
    bufs = [g.G for g in a.groups.values()] + [a.head_grad] + ([a.small_grads] if a.small_grads.numel() else [])
    bufs += [p.grad for p in a.other_params]
    hs = [comm.all_reduce_sum(b) for b in bufs]
    for h in hs:
        h.wait()
    inv = 1.0 / comm.world
    for b in bufs:
        b.mul_(inv)


def clip_gradients(model, max_norm: float = 1.0) -> torch.Tensor:
    a = model.arena
    bufs = [g.G for g in a.groups.values()] + [a.head_grad] + ([a.small_grads] if a.small_grads.numel() else [])
    bufs += [p.grad for p in a.other_params]
    total = torch.sqrt(sum(b.float().pow(2).sum() for b in bufs))
    coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
    for b in bufs:
        b.mul_(coef.to(b.dtype))
    return total


def distillation_loss(student_logits, teacher_logits, targets, mtp_loss, mtp_weight, alpha, T, label_smoothing=0.0):
    """(1 - alpha) (CE + mtp_weight * mtp) + alpha T^2 KL(student/T || teacher/T)   (unlimited/train.py:1631-1656)"""
    s = student_logits.reshape(-1, student_logits.size(-1)).float()
    t = teacher_logits.reshape(-1, teacher_logits.size(-1)).float()
    y = targets.reshape(-1)
    mask = y != -1
    ce = F.cross_entropy(s, y, label_smoothing=label_smoothing, ignore_index=-1)
    kl = F.kl_div(F.log_softmax(s[mask] / T, dim=-1), F.log_softmax(t[mask] / T, dim=-1), reduction="batchmean",
                  log_target=True) * (T ** 2)
    normal = ce + (mtp_weight * mtp_loss if mtp_loss is not None else 0.0)
    return (1 - alpha) * normal + alpha * kl


@torch.no_grad()
def target_probabilities(model, loader, steps: int) -> torch.Tensor:
    """p(ground truth) per token over `steps` batches of the fitness loader -> flat fp32 vector."""
    out = []
    it = iter(loader)
    for _ in range(steps):
        x, y, _ = next(it)
        rows = model(x, y, loss_reduction="none").view(-1).float()
        out.append(torch.exp(-rows))
    return torch.cat(out) if out else torch.zeros(0, device=model.get_device())


class UnlimitedTrainer:
    """Runs this node's chain of snapshots, then (all nodes) selection and ensemble evaluation."""

    def __init__(self, cfg: TrainConfig, info: Optional[DistInfo] = None, node_overrides: Optional[Dict[int, dict]] = None,
                 overlap_grad_reduce: bool = True):
        self.info = info or init_distributed(timeout_s=3 * 3600)     # nodes run unsynchronised for hours
        info = self.info
        self.device = info.device
        gpn = min(cfg.gpus_per_node, info.world_size)
        self.n_nodes = max(1, info.world_size // gpn)
        self.node_rank = info.rank // gpn
        cfg = config_for_node(cfg, self.node_rank, node_overrides)
        self.cfg = c = cfg
        self.node_local = info.rank % gpn
        self.is_leader = self.node_local == 0
        self.node_group, self.leader_group = None, None
        if info.world_size > 1:
            for n in range(self.n_nodes):
                g = dist.new_group(list(range(n * gpn, (n + 1) * gpn)))
                if n == self.node_rank:
                    self.node_group = g
            self.leader_group = dist.new_group([n * gpn for n in range(self.n_nodes)])
        self.node_comm = TorchComm(self.node_group) if info.world_size > 1 else TorchComm()
        self.gpn = gpn
        per_node = c.num_models // self.n_nodes
        self.model_indices = list(range(self.node_rank * per_node, (self.node_rank + 1) * per_node))
        self.ckpt_dir = os.path.join(c.checkpoint_base, c.run_name or "unlimited")
        if self.is_leader:
            os.makedirs(self.ckpt_dir, exist_ok=True)
        torch.manual_seed(c.seed + self.node_rank)
        self.model = build_model(c.model, self.device, seed=c.seed + self.node_rank, world_size=1)
        self.groups = build_param_groups(self.model, c)
        self.optimizer = ShardedMuonAdamW(self.model, self.groups, _Single())
        self.train_path = c.input_bin or os.path.join(c.data_dir, "fineweb_train.pt")
        self.val_path = c.input_val_bin or os.path.join(c.data_dir, "fineweb_val.pt")
        T = c.model.sequence_len
        self.loader = EnsembleTokenLoader(self.train_path, c.device_batch_size, T, device=self.device,
                                          seed=c.seed + self.node_rank, rank=self.node_local, world_size=gpn,
                                          fitness_tokens=c.fitness_tokens)
        self.plan = CyclePlan(c, len(self.model_indices), self.loader.total_tokens, c.device_batch_size * T * gpn)
        self.reducer = OverlappedAllReduce(self.model, self.node_comm) if (overlap_grad_reduce and self.node_comm.active) else None
        self.teacher = None
        self.pgt: Dict[int, torch.Tensor] = {}
        self.results: List[dict] = []
        self.cycle, self.step = 0, 0
        self.token_bytes = None
        self.timing = {"training": 0.0, "val_eval": 0.0, "pgt_caching": 0.0, "ensemble_eval": 0.0, "selection": 0.0}

    # ------------------------------------------------------------------ persistence
    def _snapshot_path(self, idx):
        return os.path.join(self.ckpt_dir, f"model_{idx}.pt")

    def _resume_path(self):
        return os.path.join(self.ckpt_dir, f"resume_node_{self.node_rank}.pt")

    def save_snapshot(self, idx):
        if self.is_leader:
            sd = {k: v.detach().to(torch.bfloat16).cpu() for k, v in self.model.state_dict().items()}
            torch.save(sd, self._snapshot_path(idx))
        self.node_comm.barrier()

    def save_resume(self):
        if not self.is_leader:
            return
        torch.save({"cycle": self.cycle, "step": self.step, "model": {n: p.data.float().cpu() for n, p in self.model.named_parameters()},
                    "optimizer": self.optimizer.state_dict(), "results": self.results,
                    "pgt": {k: v.cpu() for k, v in self.pgt.items()}, "signature": self.plan.signature(),
                    "flags": {"dupe_active": self.model._dupe_layers is not None}}, self._resume_path())

    def try_resume(self) -> bool:
        c = self.cfg
        if not c.resume or not os.path.exists(self._resume_path()):
            return False
        st = torch.load(self._resume_path(), map_location="cpu", weights_only=False)
        if st["signature"] != self.plan.signature():
            raise RuntimeError("resume file was written with a different batch-size schedule")
        load_named_params(self.model, st["model"])
        self.optimizer.load_state_dict(st["optimizer"])
        self.cycle, self.step, self.results = st["cycle"], st["step"], st["results"]
        self.pgt = {k: v.to(self.device) for k, v in st["pgt"].items()}
        if self.cycle > 0:
            self._load_teacher(self.model_indices[self.cycle - 1])
        # every node must resume at the same point of its chain, else the final all-node phases would deadlock
        if self.leader_group is not None and self.is_leader and self.n_nodes > 1:
            mine = torch.tensor([self.cycle, self.step], device=self.device)
            allp = [torch.zeros_like(mine) for _ in range(self.n_nodes)]
            dist.all_gather(allp, mine, group=self.leader_group)
            if any(not torch.equal(a, mine) for a in allp):
                raise RuntimeError(f"nodes disagree on the resume point: {[a.tolist() for a in allp]}")
        return True

    def _load_teacher(self, idx):
        if self.teacher is None:
            self.teacher = build_model(self.cfg.model, self.device, seed=None, world_size=1)
            for p in self.teacher.parameters():
                p.requires_grad_(False)
            self.teacher.eval()
        sd = torch.load(self._snapshot_path(idx), map_location="cpu", weights_only=True)
        load_named_params(self.teacher, {k: v for k, v in sd.items()})

    # ------------------------------------------------------------------ evaluation helpers
    def _val_loader(self):
        c = self.cfg
        return TokenLoader(self.val_path, c.device_batch_size, c.model.sequence_len, device=self.device,
                           rank=self.node_local, world_size=self.gpn, prefetch=False)

    def evaluate(self, model=None):
        c = self.cfg
        model = model or self.model
        if self.token_bytes is None:
            self.token_bytes = default_token_bytes(self.device, c.model.vocab_size)
        steps = max(1, c.eval_tokens // (c.device_batch_size * c.model.sequence_len * self.gpn))
        was = model.training
        model.eval()
        out = evaluate_bpb(model, self._val_loader(), steps, self.token_bytes, self.node_comm if self.gpn > 1 else None)
        model.train(was)
        return out

    def cache_pgt(self, idx):
        """p(ground truth) of the current weights on the fitness slice, sharded over the node's GPUs, gathered."""
        c = self.cfg
        fl = EnsembleTokenLoader(self.train_path, 4, c.model.sequence_len, device=self.device, seed=0, rank=self.node_local,
                                 world_size=self.gpn, fitness_tokens=c.fitness_tokens, fitness_only=True, prefetch=False)
        steps = min(c.pgt_steps, fl.num_steps)
        self.model.eval()
        p = target_probabilities(self.model, fl, steps)
        self.model.train()
        if self.gpn > 1:
            parts = [torch.empty_like(p) for _ in range(self.gpn)]
            dist.all_gather(parts, p, group=self.node_group)
            p = torch.cat(parts)
        self.pgt[idx] = p

    # ------------------------------------------------------------------ one training step of the current cycle
    def train_step(self, cyc: int, step_in_cycle: int, distilling: bool):
        c, model = self.cfg, self.model
        accum = self.plan.grad_accums[cyc]
        loss_t = None
        for micro in range(accum):
            x, y, _ = next(self.loader)
            if self.reducer is not None and micro == accum - 1:
                self.reducer.arm()           # reductions of finished layers start under this micro-batch's backward
            if distilling:
                s_logits, mtp_loss = model(x, y, distill=True)
                with torch.no_grad():
                    t_logits = self.teacher(x)
                loss = distillation_loss(s_logits, t_logits, y, mtp_loss, model.mtp_weight, c.distill_alpha,
                                         c.distill_temperature, c.model.label_smoothing)
            else:
                loss, _ = model(x, y, label_smoothing=c.model.label_smoothing)
            loss_t = loss.detach()
            (loss / accum).backward()
        if self.reducer is not None:
            self.reducer.finish()
        else:
            allreduce_gradients(model, self.node_comm)
        clip_gradients(model, 1.0)
        L = self.plan.lengths[cyc]
        lrm, wdm = self.plan.lr_multiplier(step_in_cycle, L), self.plan.wd_multiplier(step_in_cycle, L)
        for g in self.groups:
            g["lr"] = g["initial_lr"] * lrm
            g["weight_decay"] = g["initial_wd"] * wdm
            if g["kind"] == "muon":
                g["momentum"] = c.muon_momentum
        self.optimizer.step()
        model.zero_grad_arena()
        self.step += 1
        return loss_t

    # ------------------------------------------------------------------ the chain
    def run(self):
        c = self.cfg
        n_cycles = len(self.model_indices)
        if not self.try_resume():
            self.cycle, self.step = 0, 0
        if c.dupe_after_n_models <= self.cycle:
            self.model.set_dupe_layers(c.dupe_layers_start, c.dupe_layers_end, c.dupe_loops)
        self.model.train()
        smooth = 0.0
        while self.cycle < n_cycles:
            cyc = self.cycle
            idx = self.model_indices[cyc]
            if self.model._dupe_layers is None and cyc >= c.dupe_after_n_models:
                self.model.set_dupe_layers(c.dupe_layers_start, c.dupe_layers_end, c.dupe_loops)
            distilling = self.teacher is not None and cyc >= c.distill_after_cycles
            t0 = time.time()
            for s in range(self.plan.lengths[cyc]):
                loss = self.train_step(cyc, s, distilling)
                if c.max_steps >= 0 and self.step >= c.max_steps:
                    break
                if s % 10 == 0 and self.is_leader:
                    smooth = float(loss)
                    print(f"[node {self.node_rank}] cycle {cyc} model {idx} step {s}/{self.plan.lengths[cyc]} loss {smooth:.4f}"
                          f"{' [distill]' if distilling else ''}", flush=True)
            if self.device.type == "cuda":
                torch.cuda.synchronize()
            self.timing["training"] += time.time() - t0
            t0 = time.time()
            bpb, vloss = self.evaluate()
            self.timing["val_eval"] += time.time() - t0
            t0 = time.time()
            self.cache_pgt(idx)
            self.timing["pgt_caching"] += time.time() - t0
            self.save_snapshot(idx)
            self.results.append({"model": idx, "cycle": cyc, "val_loss": vloss, "val_bpb": bpb})
            if self.is_leader:
                print(f"[node {self.node_rank}] model {idx}: val loss {vloss:.6f} bpb {bpb:.6f}", flush=True)
            self._load_teacher(idx)
            self.cycle += 1
            if self.cycle < n_cycles:
                perturb_weights(self.model, perturb_scale(c, cyc, n_cycles), seed=c.seed * 7919 + idx,
                                comm=self.node_comm if self.gpn > 1 else None)
            self.save_resume()
            if c.max_steps >= 0 and self.step >= c.max_steps:
                break
        return self.finish()

    # ------------------------------------------------------------------ selection + ensemble evaluation
    def finish(self):
        c = self.cfg
        t0 = time.time()
        ids = sorted(self.pgt.keys())
        P = torch.stack([self.pgt[i] for i in ids]) if ids else torch.zeros(0, 0, device=self.device)
        if self.n_nodes > 1 and self.leader_group is not None:
            # leaders exchange their rows: every node contributes `per_node` rows of the same width
            full = torch.zeros(c.num_models, P.size(1), device=self.device)
            if self.is_leader:
                for r, i in enumerate(ids):
                    full[i] = P[r]
                dist.all_reduce(full, group=self.leader_group)
            dist.broadcast(full, src=self.node_rank * self.gpn, group=self.node_group)
            P, ids = full, list(range(c.num_models))
        sel = select_members(P, c.k_sweep, c.grad_opt_steps, c.grad_lr, seed=c.seed) if len(ids) else None
        self.timing["selection"] += time.time() - t0
        out = {"models": self.results, "selection": {}, "ensemble": {}, "timing": self.timing}
        if sel is not None:
            t0 = time.time()
            mixtures = {}
            for k, s in sel.by_k.items():
                members = [ids[m] for m in s.members]
                weights = s.weights if c.grad_weighted_eval else [1.0 / len(members)] * len(members)
                mixtures[k] = (members, weights)
                out["selection"][k] = {"members": members, "weights": s.weights, "fit_loss": s.fit_loss}
            for k, (bpb, loss) in self.evaluate_ensembles(mixtures).items():
                out["ensemble"][k] = {"val_loss": loss, "val_bpb": bpb}
                print0(f"ensemble K={k}: members {mixtures[k][0]} val loss {loss:.6f} bpb {bpb:.6f}")
            self.timing["ensemble_eval"] += time.time() - t0
        if self.info.rank == 0:
            with open(os.path.join(self.ckpt_dir, "progress.json"), "w") as f:
                json.dump({"individual_models": self.results, **out}, f, indent=2)
            if c.save_result:
                with open(c.save_result, "w") as f:
                    json.dump(self.result_record(out), f, indent=2)
        return out

    def result_record(self, out):
        """The result file of the reference (unlimited/train.py:2161-2196): configuration, distillation and
        perturbation settings, per-node overrides, every snapshot's validation numbers and the K sweep."""
        c, m = self.cfg, self.cfg.model
        rec = {
            "config": {"n_layer": m.n_layer, "n_embd": m.n_embd, "n_head": m.n_head, "total_batch_size": c.total_batch_size,
                       "epochs_per_cycle": c.epochs_per_cycle, "num_models": c.num_models,
                       "dupe_layers": f"{c.dupe_layers_start}-{c.dupe_layers_end}", "dupe_after_n_models": c.dupe_after_n_models},
            "chain_distillation": {"alpha": c.distill_alpha, "temperature": c.distill_temperature,
                                   "after_cycles": c.distill_after_cycles, "teacher": "last_snapshot"},
            "weight_perturbation": {"perturb_scale_max": c.perturb_scale, "perturb_scale_min": c.perturb_scale_min},
            "node_overrides": getattr(c, "node_overrides", {}),
            "individual_models": self.results,
            "timing": self.timing,
        }
        if out["ensemble"]:
            rec["grad_sweep"] = [{"k": k, "selected_models": [i + 1 for i in out["selection"][k]["members"]],
                                  "weights": out["selection"][k]["weights"], "val_bpb": out["ensemble"][k]["val_bpb"],
                                  "val_loss": out["ensemble"][k]["val_loss"], "fit_loss": out["selection"][k]["fit_loss"]}
                                 for k in sorted(out["ensemble"])]
            best = max(out["ensemble"])          # the largest K is the canonical final ensemble
            rec["final_ensemble_bpb"] = out["ensemble"][best]["val_bpb"]
            rec["final_ensemble_loss"] = out["ensemble"][best]["val_loss"]
        return rec

    @torch.no_grad()
    def evaluate_ensembles(self, mixtures: Dict[int, tuple]):
        """Validation loss / BPB of several weighted probability mixtures of snapshots at once
        (unlimited/train.py:1036-1148 evaluates one mixture per call, keeping up to 64 models resident per GPU).
        Here every snapshot that occurs in any mixture is loaded and run ONCE, by the rank it is dealt to; its
        per-token p(target) over the evaluation batches is kept on the host (4 bytes per token), and each mixture is a
        weighted sum of those vectors followed by one all-reduce. One model is resident per GPU at a time.
        mixtures: {K: (member indices, weights)} -> {K: (bpb, loss)}"""
        c = self.cfg
        world, rank = self.info.world_size, self.info.rank
        if self.token_bytes is None:
            self.token_bytes = default_token_bytes(self.device, c.model.vocab_size)
        steps = max(1, c.eval_tokens // (c.device_batch_size * c.model.sequence_len))
        loader = TokenLoader(self.val_path, c.device_batch_size, c.model.sequence_len, device=self.device, prefetch=False)
        batches = [next(loader)[:2] for _ in range(steps)]
        union = sorted({m for members, _ in mixtures.values() for m in members})
        mine = union[rank::world]
        probs = {}
        for m in mine:
            self._load_teacher(m)
            probs[m] = torch.stack([torch.exp(-self.teacher(x, y, loss_reduction="none").reshape(-1).float()) for x, y in batches]).cpu()
        from .evaluate import _Tally
        out = {}
        for k, (members, weights) in mixtures.items():
            acc = torch.zeros(steps, batches[0][1].numel(), device=self.device)
            for m, w in zip(members, weights):
                if m in probs:
                    acc.add_(probs[m].to(self.device), alpha=float(w))
            if world > 1:
                dist.all_reduce(acc)
            tally = _Tally(self.device, self.token_bytes)
            for i, (_, y) in enumerate(batches):
                tally.add(-torch.log(acc[i].clamp_min(1e-40)), y)
            out[k] = tally.result(None)          # every rank holds the full mixture after the all-reduce
        return out

    def evaluate_ensemble(self, members: List[int], weights: List[float]):
        """One mixture: (bpb, loss)."""
        return self.evaluate_ensembles({0: (members, weights)})[0]
