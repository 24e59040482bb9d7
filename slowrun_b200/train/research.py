"""Trainers of the two research forks, on the package's training loop.

* `HybridTrainer`   research/hybrid_attn/train.py: softmax / linear-attention hybrid model, optional gradient clipping
                    (:1575-1576), CPU-side weight EMAs started late in the run and a 0.7 / 0.3 blend of final and
                    averaged weights evaluated at the end (:239-269, 1593-1601, 1676-1693), average of the last epoch
                    checkpoints (:262-270, 1695-1712), section timers around the linear-attention stages (:179-233),
                    both Muon variants and both Newton-Schulz coefficient tables (:932-1019), and a start-up probe of
                    the recurrent token-mixer path (:1386-1420).
* `UniversalTrainer` research/universal_transformer/train.py: depth-shared model whose active depth grows at given
                    steps (:1173, 1219-1230); parameters of layers that do not run yet receive no gradient and are
                    left alone by the optimizer (:659-755), every scheduled depth is exercised once before training
                    starts and the weights are re-initialised afterwards (:1053-1075).

Both reuse `Trainer` (data order, gradient accumulation, sharded Muon/AdamW, schedules, evaluation, logging); the
models run on plain PyTorch ops under bf16 autocast on a GPU, without CUDA-graph capture.
"""
from __future__ import annotations

import contextlib
import time
from typing import Dict, List, Optional

import torch

from ..config import TrainConfig
from ..parallel.comm import print0
from .checkpoint import load_named_params, named_param_snapshot
from .trainer import Trainer


class SectionProfiler:
    """Wall-clock timers around named sections, each bracketed by a device synchronisation (so the numbers are only
    meaningful in eager execution, and cost throughput: off unless asked for)."""

    def __init__(self, enabled=False, synchronize=None):
        self.enabled = enabled
        self._sync = synchronize or (lambda: None)
        self.stats: Dict[str, List[float]] = {}

    @contextlib.contextmanager
    def section(self, name):
        if not self.enabled:
            yield
            return
        self._sync()
        t0 = time.perf_counter()
        try:
            yield
        finally:
            self._sync()
            rec = self.stats.setdefault(name, [0.0, 0])
            rec[0] += time.perf_counter() - t0
            rec[1] += 1

    def summary(self) -> Dict[str, dict]:
        total = sum(t for t, _ in self.stats.values())
        if total <= 0:
            return {}
        return {k: {"total_sec": t, "count": n, "avg_ms": 1000.0 * t / max(n, 1), "pct_total": 100.0 * t / total}
                for k, (t, n) in sorted(self.stats.items(), key=lambda kv: -kv[1][0])}

    def lines(self):
        return [f"  {k}: {v['avg_ms']:.2f}ms avg over {v['count']} calls ({v['pct_total']:.1f}%)" for k, v in self.summary().items()]


class EMATracker:
    """Exponential moving average of the weights, kept in fp32 on the host."""

    def __init__(self, model, decay: float):
        self.decay = decay
        self.shadow = {n: p.data.float().cpu().clone() for n, p in model.named_parameters()}
        self.num_updates = 0

    @torch.no_grad()
    def update(self, model):
        self.num_updates += 1
        for n, p in model.named_parameters():
            self.shadow[n].lerp_(p.data.float().cpu(), 1 - self.decay)


def clip_local_grad_norm_(model, max_norm: float) -> torch.Tensor:
    """Scale this rank's accumulated gradients so that their global 2-norm is at most `max_norm` (before they are
    reduced across ranks, as in the fork). Returns the norm."""
    grads = [p.grad for p in model.parameters() if p.grad is not None]
    head = getattr(model.arena, "head_grad", None) if getattr(model, "arena", None) is not None else None
    if head is not None and all(head.data_ptr() != g.data_ptr() for g in grads):
        grads.append(head)
    norm = torch.sqrt(sum(g.float().square().sum() for g in grads))
    factor = (max_norm / (norm + 1e-6)).clamp(max=1.0)
    for g in grads:
        g.mul_(factor.to(g.dtype))
    return norm


class _ResearchTrainer(Trainer):
    def __init__(self, cfg: TrainConfig, info=None, quiet=False):
        cfg.cuda_graphs = False
        super().__init__(cfg, info, quiet)

    def forward_context(self):
        if self.device.type == "cuda":
            return torch.autocast(device_type="cuda", dtype=torch.bfloat16)
        return contextlib.nullcontext()


class HybridTrainer(_ResearchTrainer):
    def __init__(self, cfg: TrainConfig, spec, grad_clip: float = 0.0, ema_decays=(0.95,), ema_start_frac: float = 0.90,
                 checkpoint_avg: int = 0, info=None, quiet=False):
        self.spec = spec
        self.grad_clip = float(grad_clip)
        self.ema_decays = [float(d) for d in ema_decays]
        self.checkpoint_avg = int(checkpoint_avg)
        cfg.track = "hybrid"
        super().__init__(cfg, info, quiet)
        sync = torch.cuda.synchronize if self.device.type == "cuda" else None
        self.profiler = SectionProfiler(spec.profile, sync)
        self.model.set_profiler(self.profiler)
        self.ema_start_step = round(ema_start_frac * self.sched.N)
        self.ema_trackers: List[EMATracker] = []
        self.late_checkpoints: List[dict] = []
        self.last_grad_norm: Optional[float] = None
        if spec.use_recurrent:
            self.probe_recurrent_path()

    def model_factory(self):
        from ..models.hybrid import HybridGPT
        return lambda mc: HybridGPT(mc, self.spec)

    def probe_recurrent_path(self):
        """Run the token-by-token path forward and backward on a few tokens before committing hours to it."""
        from ..ops.linear_attention import gated_delta_rule
        dev = self.device
        q, k = (torch.randn(1, 4, 2, 64, device=dev, requires_grad=True) for _ in range(2))
        v = torch.randn(1, 4, 2, 16, device=dev, requires_grad=True)
        g = -torch.rand(1, 4, 2, device=dev)
        beta = torch.rand(1, 4, 2, device=dev)
        gated_delta_rule(q, k, v, g, beta, impl="recurrent").float().sum().backward()
        if not all(torch.isfinite(t.grad).all() for t in (q, k, v)):
            raise RuntimeError("the recurrent gated-delta-rule path produced non-finite gradients on the start-up probe")

    def before_optimizer_step(self):
        if self.grad_clip > 0:
            self.last_grad_norm = float(clip_local_grad_norm_(self.model, self.grad_clip))

    def after_optimizer_step(self):
        step = self.step + 1
        if self.ema_decays and step >= self.ema_start_step and step % 10 == 0:
            if not self.ema_trackers:
                print0(f"Initializing {len(self.ema_decays)} EMA tracker(s) at step {step}")
                self.ema_trackers = [EMATracker(self.model, d) for d in self.ema_decays]
            for ema in self.ema_trackers:
                ema.update(self.model)

    def on_epoch_end(self, epoch, val_bpb, val_loss):
        if self.checkpoint_avg > 0:
            self.late_checkpoints.append(named_param_snapshot(self.model))
            del self.late_checkpoints[:-self.checkpoint_avg]

    def _load(self, weights):
        load_named_params(self.model, weights)

    def post_training(self, log, best):
        min_bpb, min_loss = best
        final = named_param_snapshot(self.model) if (self.ema_trackers or len(self.late_checkpoints) >= 2) else None
        alpha = 0.7
        for ema in self.ema_trackers:
            print0(f"\n--- Evaluating EMA blend (decay={ema.decay}, {ema.num_updates} updates) ---")
            self._load({n: alpha * final[n] + (1 - alpha) * ema.shadow[n] for n in final})
            bpb, loss = self.evaluate()
            print0(f"Blend({alpha:.1f}*final+{1 - alpha:.1f}*EMA {ema.decay}): Val BPB: {bpb:.6f} | Val Loss: {loss:.6f}")
            log.metrics({f"ema_blend_{ema.decay}/bpb": bpb, f"ema_blend_{ema.decay}/loss": loss})
            if loss < min_loss:
                min_loss, min_bpb = loss, bpb
                print0(f"  ** New best! (from blend {alpha:.1f}/{1 - alpha:.1f} with EMA {ema.decay})")
            self._load(final)
        if len(self.late_checkpoints) >= 2:
            n = len(self.late_checkpoints)
            print0(f"\n--- Evaluating checkpoint average ({n} checkpoints) ---")
            self._load({k: sum(ck[k] for ck in self.late_checkpoints) / n for k in self.late_checkpoints[0]})
            bpb, loss = self.evaluate()
            print0(f"Checkpoint avg: Val BPB: {bpb:.6f} | Val Loss: {loss:.6f}")
            log.metrics({"ckpt_avg/bpb": bpb, "ckpt_avg/loss": loss})
            if loss < min_loss:
                min_loss, min_bpb = loss, bpb
                print0("  ** New best! (from checkpoint averaging)")
            self._load(final)
        if self.profiler.enabled:
            print0("Section timings:")
            for line in self.profiler.lines():
                print0(line)
        return min_bpb, min_loss


class UniversalTrainer(_ResearchTrainer):
    def __init__(self, cfg: TrainConfig, model_config, info=None, quiet=False, exercise_depths: bool = True):
        self.uconfig = model_config
        cfg.track = "universal"
        cfg.model.sequence_len = model_config.sequence_len
        super().__init__(cfg, info, quiet)
        self.schedule = self.model.schedule
        self._stage = 0
        if exercise_depths:
            self.exercise_scheduled_depths()
        self._sync_active_set()

    def model_factory(self):
        from ..models.research import UniversalGPT
        return lambda mc: UniversalGPT(self.uconfig)

    def _sync_active_set(self):
        self.optimizer.set_inactive(self.model.inactive_parameters())
        self.flops_per_token = self.model.estimate_flops()

    def exercise_scheduled_depths(self):
        """One forward / backward / optimizer step and one evaluation forward at every depth of the schedule on the
        first batch, so that a depth that cannot run fails now and not hours in; then the weights are initialised
        again and the optimizer state is rebuilt."""
        from ..optim.muon_adamw import ShardedMuonAdamW
        model = self.model
        for depth in sorted({d for _, d in self.schedule}):
            model.set_active_layers(depth)
            self.optimizer.set_inactive(model.inactive_parameters())
            model.train()
            with self.forward_context():
                loss = model(self.x, self.y)
            loss.backward()
            self.optimizer.step()
            model.zero_grad_arena()
            model.eval()
            with torch.no_grad(), self.forward_context():
                model(self.x, self.y, loss_reduction="none")
        torch.manual_seed(42)
        model.init_weights()
        model.arena.refresh_shadows()
        model.set_active_layers(self.schedule[0][1])
        model.train()
        self.optimizer = ShardedMuonAdamW(model, self.param_groups, self.comm)

    def after_optimizer_step(self):
        step = self.step + 1
        if self._stage + 1 < len(self.schedule) and step >= self.schedule[self._stage + 1][0]:
            self._stage += 1
            self.model.set_active_layers(self.schedule[self._stage][1])
            self._sync_active_set()
            print0(f"Step {step:05d} | n_layer -> {self.model.active_n_layer}")
