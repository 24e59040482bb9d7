"""Training driver for the limited, two-hour and tiny tracks.

`Trainer.train_step()` is one optimizer step: `grad_accum` micro-batches of forward/backward with local fp32
gradient accumulation, the schedules, then the sharded optimizer step (the only place gradients cross GPUs), as in
the reference loop (train.py:1146-1254, tiny/train.py:1400-1470). `Trainer.fit()` adds evaluation at epoch
boundaries, the checkpoint ring, dupe-layer / window / recurrence switches, early stopping and the post-training
averaging passes. Log lines keep the reference's format so existing parsers work.
"""
from __future__ import annotations

import gc
import json
import math
import os
import shutil
import sys
import time
from typing import Optional

import torch

from ..config import TrainConfig, MAX_SEQ_LEN
from ..data.loader import TokenLoader
from ..models.gpt import build_model
from ..optim.groups import build_param_groups
from ..optim.muon_adamw import ShardedMuonAdamW
from ..ops import _lib
from ..parallel.comm import DistInfo, TorchComm, init_distributed, print0
from ..utils.debug import nvtx_range
from ..utils.logging import RunLogger
from .checkpoint import (CheckpointRing, WeightEMA, average_checkpoints_into, full_state_exists, load_full_state,
                         recency_weights, save_full_state)
from .evaluate import default_token_bytes, evaluate_bpb, evaluate_prob_avg
from .schedules import Schedules, parse_window_schedule, window_stage_for_epoch


def make_comm(cfg: TrainConfig, info: DistInfo):
    """Collective backend: peer-memory kernels on multi-GPU CUDA jobs unless --comm nccl, else torch.distributed."""
    if info.world_size > 1 and info.device.type == "cuda" and cfg.comm in ("auto", "fused"):
        try:
            from ..parallel.fused import FusedComm
            return FusedComm()
        except Exception as e:  # noqa: BLE001 - fall back to the library path, loudly
            if cfg.comm == "fused":
                raise
            print0(f"[comm] peer-memory collectives unavailable ({type(e).__name__}: {e}); using NCCL")
    return TorchComm()


class Trainer:
    # tracks whose post-training step is the probability average over the last epoch checkpoints on disk
    LOGIT_AVG_TRACKS = ("limited", "two_hour", "universal")
    # tracks that replay decoder layers from `dupe_start_epoch` on
    DUPE_TRACKS = ("limited", "two_hour", "hybrid")

    def model_factory(self):
        """Constructor of the model (`factory(model_config) -> GPT-like module`), or None for the package's GPT."""
        return None

    def forward_context(self):
        """Context the forward pass runs in (research models on plain PyTorch ops use bf16 autocast on a GPU)."""
        import contextlib
        return contextlib.nullcontext()

    def before_optimizer_step(self):
        """Hook: gradients of the step are complete (local, not yet reduced across ranks)."""

    def after_optimizer_step(self):
        """Hook: parameters were updated; `self.step` still holds the index of the step just taken."""

    def on_epoch_end(self, epoch, val_bpb, val_loss):
        """Hook: `epoch` was just evaluated (called on every rank)."""

    def post_training(self, log, best):
        """Hook after the last step: `best` = (min_bpb, min_loss); returns the possibly improved pair."""
        return best

    def __init__(self, cfg: TrainConfig, info: Optional[DistInfo] = None, quiet: bool = False):
        self.cfg = cfg
        self.info = info or init_distributed()
        info = self.info
        self.device = info.device
        self.master = info.rank == 0
        self.quiet = quiet
        c = cfg
        seed = c.seed if c.track == "unlimited" else 42
        self.stream = None
        if self.device.type == "cuda" and c.cuda_graphs:
            # Everything runs on one non-default stream from the first forward on: autograd's per-parameter
            # gradient accumulators remember the stream they were created on, and a CUDA-graph capture must not touch
            # the default stream.
            self.stream = torch.cuda.Stream(device=self.device)
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            torch.cuda.set_stream(self.stream)
        self.comm = make_comm(c, info)
        self.model = build_model(c.model, self.device, seed=seed, world_size=info.world_size,
                                 alloc=self.comm.alloc if getattr(self.comm, "fused", False) else None,
                                 factory=self.model_factory())
        self.param_groups = build_param_groups(self.model, c)
        self.optimizer = ShardedMuonAdamW(self.model, self.param_groups, self.comm, wire_dtype=c.wire_dtype)
        train_path = c.input_bin or os.path.join(c.data_dir, "fineweb_train.pt")
        self.val_path = c.input_val_bin or os.path.join(c.data_dir, "fineweb_val.pt")
        T = c.model.sequence_len
        self.train_loader = TokenLoader(train_path, c.device_batch_size, T, device=self.device,
                                        doc_shuffle=not c.no_doc_shuffle, rank=info.rank, world_size=info.world_size)
        self.tokens_per_epoch = self.train_loader.total_tokens
        tokens_per_fwdbwd = c.device_batch_size * T * info.world_size
        assert c.total_batch_size % tokens_per_fwdbwd == 0, "total batch must be a multiple of B*T*world"
        self.grad_accum = c.total_batch_size // tokens_per_fwdbwd
        self.sched = Schedules(c, self.tokens_per_epoch)
        self.window_schedule = parse_window_schedule(c.window_schedule, T) if c.track == "two_hour" else ()
        self.step = 0
        self.current_epoch = 1
        self.smooth_loss = 0.0
        self.dupe_active = False
        self.x, self.y, self.current_epoch = next(self.train_loader)
        self._pending_epoch = self.current_epoch
        self.flops_per_token = self.model.estimate_flops()
        self.token_bytes = None
        self.ema = None
        if c.track == "tiny" and c.update_ema_every > 0:
            self.ema = WeightEMA(self.model, c.ema_decay_per_epoch, c.update_ema_every, self.sched.steps_per_epoch)
        st = window_stage_for_epoch(self.window_schedule, self.current_epoch)
        if st is not None:
            self.model.set_window_sizes(st.short_window, st.long_window)
        self.model.train()
        self.h2d_bytes_per_step = self.train_loader.h2d_bytes_per_batch * self.grad_accum
        self.d2h_bytes_per_step = 4
        # CUDA graphs of one micro-batch (forward + backward), keyed by everything that changes the kernel sequence
        self._graphs = {}
        self._graph_key = None
        self._eager_micro = 0
        self.use_graphs = bool(c.cuda_graphs) and self.device.type == "cuda"
        # gradient reduction under the last backward pass (peer-memory optimizer only): `--overlap-backward` or
        # SLOWRUN_OVERLAP_BACKWARD=1. Off by default: with 8-64 micro-batches per step the pulls it hides are 1-2 % of a
        # step, about what the eagerly launched last micro-batch gives back (measured at 2 GPUs: 100.1 k tokens/s with,
        # 100.7 k without).
        want = os.environ.get("SLOWRUN_OVERLAP_BACKWARD")
        want = c.overlap_backward if want is None else want != "0"
        self.overlap_backward = bool(want) and self.optimizer.can_overlap_backward()

    # ------------------------------------------------------------------ one optimizer step
    def _maybe_switch_structure(self):
        c = self.cfg
        if c.track in self.DUPE_TRACKS and not self.dupe_active and self.current_epoch >= c.dupe_start_epoch:
            self.model.set_dupe_layers(c.dupe_layers_start, c.dupe_layers_end, c.dupe_loops)
            self.dupe_active = True
            self.flops_per_token = self.model.estimate_flops()
            if not self.quiet:
                print0(f"\n=== Enabling dupe-layers at epoch {self.current_epoch} ===")
                print0(f"Dupe layers {c.dupe_layers_start}-{c.dupe_layers_end - 1}: {c.dupe_loops} extra replays ({c.dupe_loops + 1} total passes)")

    def train_step(self, sync: bool = True):
        """Runs one optimizer step. Returns a dict with the (host) loss of the last micro-batch when `sync`."""
        c, model = self.cfg, self.model
        self._maybe_switch_structure()
        tiny = c.track == "tiny"
        n_iter = self.sched.num_recurrences(self.step) if tiny else None
        mtp_w = None
        if tiny and c.model.fused_mtp:
            mtp_w = torch.tensor(self.sched.mtp_weights(self.step), dtype=torch.float32, device=self.device)
        metrics = {}
        loss_t = None
        epoch = self._pending_epoch
        key = (self.dupe_active, n_iter, tuple(model.window_sizes), model.rotary.attn_scale, self.grad_accum)
        if key != self._graph_key:
            self._graph_key, self._eager_micro = key, 0
        for micro in range(self.grad_accum):
            # last micro-batch on the peer-memory path: run eagerly so that each layer's gradients can be released to
            # their owners (and pulled by them on a side stream) while the backward pass is still walking down
            overlapped = (self.overlap_backward and micro == self.grad_accum - 1 and self.optimizer.begin_backward_overlap())
            rng = nvtx_range("micro_step").__enter__()
            graph = self._graphs.get(key) if (self.use_graphs and not overlapped) else None
            if graph is None and self.use_graphs and not overlapped and self._eager_micro >= 3:
                graph = self._capture(key, tiny, n_iter, mtp_w)
            if graph is not None:
                graph["x"].copy_(self.x)
                graph["y"].copy_(self.y)
                if mtp_w is not None:
                    graph["mtp_w"].copy_(mtp_w)
                graph["g"].replay()
                _lib.launch_count += graph["launches"]      # kernels replayed from the graph
                loss_t, metrics = graph["loss"], graph["metrics"]
            else:
                with self.forward_context():
                    out = model(self.x, self.y, num_iterations=n_iter, mtp_weights=mtp_w) if tiny else model(self.x, self.y)
                loss, metrics = out if isinstance(out, tuple) else (out, {})
                loss_t = loss.detach()
                (loss / self.grad_accum).backward()
                self._eager_micro += 1
                if overlapped:
                    self.optimizer.finish_backward_overlap()
            rng.__exit__(None, None, None)
            self.x, self.y, epoch = next(self.train_loader)
        self._pending_epoch = epoch
        self.before_optimizer_step()
        self.sched.apply(self.param_groups, self.step)
        with nvtx_range("optimizer_step"):
            self.optimizer.step()
        if getattr(self.optimizer, "fused", False):
            # a device-side barrier that gave up leaves the status word set and every consumer kernel of the step
            # returned without writing: stop here, before the gradients are cleared, instead of training on
            _lib.check_status(self.device)
        model.zero_grad_arena()
        if self.ema is not None:
            self.ema.maybe_update(self.step)
        self.after_optimizer_step()
        self.step += 1
        out = {"loss_tensor": loss_t, "metrics": metrics, "epoch": epoch, "num_iterations": n_iter}
        if sync:
            out["loss"] = loss_t.item()
            if self.device.type == "cuda":
                _lib.check_status(self.device)
        return out

    def _capture(self, key, tiny, n_iter, mtp_w):
        """Capture forward+backward of one micro-batch into a CUDA graph (static input buffers, gradients accumulate
        in place into the arenas). Returns None and disables graphs if the capture is refused."""
        model = self.model
        sx, sy = torch.empty_like(self.x), torch.empty_like(self.y)
        sx.copy_(self.x)
        sy.copy_(self.y)
        sw = mtp_w.clone() if mtp_w is not None else None
        g = torch.cuda.CUDAGraph()
        launches0 = _lib.launch_count
        try:
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=self.stream):
                if tiny:
                    loss = model(sx, sy, num_iterations=n_iter, mtp_weights=sw)
                    metrics = {}
                else:
                    loss, metrics = model(sx, sy)
                (loss / self.grad_accum).backward()
                loss_d = loss.detach()
                metrics = {k: v.detach() for k, v in metrics.items()}
        except Exception as e:  # noqa: BLE001
            print0(f"[graphs] capture refused ({type(e).__name__}: {e}); continuing without CUDA graphs")
            self.use_graphs = False
            torch.cuda.synchronize()
            return None
        # the capture pass itself does not execute kernels: replay once so this micro-batch is accounted for
        entry = {"g": g, "x": sx, "y": sy, "mtp_w": sw, "loss": loss_d, "metrics": metrics,
                 "launches": _lib.launch_count - launches0}
        _lib.launch_count = launches0
        self._graphs[key] = entry
        return entry

    # ------------------------------------------------------------------ stop and continue
    def save_state(self, path: str, fit_state=None):
        """Everything needed to continue this run at the current step on the same number of ranks: weights, this rank's
        optimizer shard, RNG streams, the loader position (the batch already fetched for the next step is delivered
        again), epoch / schedule flags, the weight EMA. The reference has this only for its unlimited track
        (unlimited/train.py:1897-1918)."""
        extra = {"current_epoch": self.current_epoch, "pending_epoch": self._pending_epoch, "smooth_loss": self.smooth_loss,
                 "dupe_active": self.dupe_active, "fit": fit_state or {}}
        if self.ema is not None and self.ema.ema is not None:
            extra["ema"] = {"updates": self.ema.updates, "tensors": [e.detach().cpu() for e in self.ema.ema]}
        save_full_state(path, self.model, self.optimizer, self.train_loader.state(rewind=1), self.step, extra,
                        rank=self.info.rank, world_size=self.info.world_size)
        self.comm.barrier()

    def load_state(self, path: str) -> dict:
        c = self.cfg
        st = load_full_state(path, self.model, self.optimizer, rank=self.info.rank, world_size=self.info.world_size)
        ex = st["extra"]
        self.step = int(st["step"])
        self.current_epoch, self.smooth_loss = int(ex["current_epoch"]), float(ex["smooth_loss"])
        if ex.get("dupe_active") and not self.dupe_active:
            self.model.set_dupe_layers(c.dupe_layers_start, c.dupe_layers_end, c.dupe_loops)
            self.dupe_active = True
            self.flops_per_token = self.model.estimate_flops()
        for e in range(2, self.current_epoch + 1):       # replay the window stages: each longer window rescales the rotary
            stage = window_stage_for_epoch(self.window_schedule, e)
            if stage is not None and (stage.short_window != self.model.short_window or stage.long_window != self.model.long_window):
                self.model.set_window_sizes(stage.short_window, stage.long_window, apply_yarn=True)
                self.flops_per_token = self.model.estimate_flops()
        if self.ema is not None and "ema" in ex:
            self.ema.updates = int(ex["ema"]["updates"])
            for e, saved in zip(self.ema.ema, ex["ema"]["tensors"]):
                e.copy_(saved)
        self.train_loader.restore(st["loader"])
        self.x, self.y, self._pending_epoch = next(self.train_loader)
        self._graphs, self._graph_key, self._eager_micro = {}, None, 0
        self.comm.barrier()
        return ex.get("fit", {})

    # ------------------------------------------------------------------ evaluation helpers
    def build_val_loader(self):
        c = self.cfg
        return TokenLoader(self.val_path, c.device_batch_size, c.model.sequence_len, device=self.device,
                           rank=self.info.rank, world_size=self.info.world_size, prefetch=False)

    def evaluate(self, num_iterations=None):
        c = self.cfg
        if self.token_bytes is None:
            self.token_bytes = default_token_bytes(self.device, c.model.vocab_size)
        steps = max(1, c.eval_tokens // (c.device_batch_size * c.model.sequence_len * self.info.world_size))
        self.model.eval()
        with self.forward_context():
            bpb, loss = evaluate_bpb(self.model, self.build_val_loader(), steps, self.token_bytes,
                                     self.comm if self.info.world_size > 1 else None, num_iterations=num_iterations)
        self.model.train()
        return bpb, loss

    def sync_epoch(self, epoch: int) -> int:
        if self.info.world_size > 1:
            t = torch.tensor([epoch], dtype=torch.long, device=self.device)
            self.comm.all_reduce_max(t)
            return int(t.item())
        return epoch

    # ------------------------------------------------------------------ full run
    def fit(self):
        c, info = self.cfg, self.info
        log = RunLogger(c, info, quiet=self.quiet)
        self.log = log
        log.hyperparameters(c, self.model, self.flops_per_token)
        world = info.world_size
        N = self.sched.N
        target_steps = c.max_train_steps if (c.track == "tiny" and c.max_train_steps > 0) else N
        print0(f"Batch size: {c.total_batch_size:,} tokens, grad accum: {self.grad_accum} steps")
        print0(f"Training for {c.num_epochs} epoch(s) (~{N} steps estimated)")
        print0(f"Eval set: {c.eval_tokens:,} tokens")
        min_bpb = min_loss = float("inf")
        val_bpb = val_loss = float("inf")
        bad_epochs = 0
        total_time, timed_steps, timing_start = 0.0, 0, 4
        keep = c.logit_avg if c.track in self.LOGIT_AVG_TRACKS else (c.swa_last_epochs if c.track == "tiny" else 0)
        ring_dir = c.logit_avg_dir if c.track in self.LOGIT_AVG_TRACKS else os.path.join(log.run_dir, "checkpoints")
        ring = CheckpointRing(ring_dir, keep, self.master)
        max_iters = c.model.num_iterations if c.track == "tiny" else None
        resume_path = c.resume or os.path.join(log.run_dir, "resume")
        resumed = False
        if c.resume and full_state_exists(c.resume, info.rank):
            fs = self.load_state(c.resume)
            min_bpb, min_loss = fs.get("min_bpb", min_bpb), fs.get("min_loss", min_loss)
            bad_epochs, ring.paths = fs.get("bad_epochs", 0), list(fs.get("ring_paths", []))
            resumed = True
            print0(f"Resumed from {c.resume} at step {self.step} (epoch {self.current_epoch})")
        if not c.eval_logit_avg and not resumed:
            val_bpb, val_loss = self.evaluate(max_iters)
            print0(f"Step {self.step:05d} | Val BPB: {val_bpb:.6f} | Val Loss: {val_loss:.6f}")
            log.metrics({"step": self.step, "val/bpb": val_bpb, "val/loss": val_loss})
            min_bpb, min_loss = val_bpb, val_loss
        synchronize = torch.cuda.synchronize if self.device.type == "cuda" else (lambda: None)
        while not c.eval_logit_avg and self.current_epoch <= c.num_epochs:
            if c.max_steps >= 0 and self.step >= c.max_steps:
                break
            was_dupe = self.dupe_active
            synchronize()
            t0 = time.time()
            out = self.train_step(sync=True)
            synchronize()
            dt = time.time() - t0
            if self.dupe_active and not was_dupe:
                timing_start = self.step + 3
            step = self.step
            self.smooth_loss = 0.9 * self.smooth_loss + 0.1 * out["loss"]
            debiased = self.smooth_loss / (1 - 0.9 ** step)
            tok_s = int(c.total_batch_size / dt)
            mfu = 100 * self.flops_per_token * c.total_batch_size / dt / (log.peak_flops * world)
            if step >= timing_start:
                total_time += dt
                timed_steps += 1
            eta = f" | eta: {(target_steps - step) * total_time / timed_steps / 60:.1f}m" if timed_steps > 0 else ""
            tag = " [DUPE]" if self.dupe_active else ""
            it_s = f" | iters: {out['num_iterations']}" if out["num_iterations"] is not None else ""
            print0(f"step {step:05d} ({100 * step / target_steps:.2f}%) | loss: {debiased:.6f} | dt: {dt * 1000:.2f}ms | "
                   f"tok/sec: {tok_s:,} | bf16_mfu: {mfu:.2f}%{it_s}{tag}{eta}")
            log.metrics({"step": step, "train/loss": debiased, "train/mfu": mfu, "train/tok_per_sec": tok_s,
                         **{f"train/{k}": float(v.detach()) for k, v in out["metrics"].items()}})
            epoch = self.sync_epoch(out["epoch"])
            if epoch != self.current_epoch:
                val_bpb, val_loss = self.evaluate(max_iters)
                print0(f"Step {step:05d} | Epoch {self.current_epoch} | Val BPB: {val_bpb:.6f} | Val Loss: {val_loss:.6f}")
                log.metrics({"step": step, "epoch": self.current_epoch, "val/bpb": val_bpb, "val/loss": val_loss})
                self.on_epoch_end(self.current_epoch, val_bpb, val_loss)
                stop = False
                if val_bpb < min_bpb:
                    min_bpb, min_loss, bad_epochs = val_bpb, val_loss, 0
                else:
                    bad_epochs += 1
                    if c.patience >= 0 and bad_epochs >= c.patience:
                        print0(f"Early stopping: no improvement for {c.patience} epoch(s)")
                        stop = True
                if keep > 0 and not stop:
                    path = ring.save(self.model, self.current_epoch)
                    print0(f"  Saved checkpoint {path} ({len(ring.paths)}/{keep})")
                    # only rank 0 writes (seconds for a multi-GB model); the others wait here on the host, not inside
                    # the next step's device-side barrier
                    self.comm.barrier()
                if stop:
                    break
                st = window_stage_for_epoch(self.window_schedule, epoch)
                if st is not None and (st.short_window != self.model.short_window or st.long_window != self.model.long_window):
                    self.model.set_window_sizes(st.short_window, st.long_window, apply_yarn=True)
                    self.flops_per_token = self.model.estimate_flops()
                    print0(f"Updated window stage for epoch {epoch}: short={st.short_window}, long={st.long_window}, "
                           f"yarn_scale={self.model.rotary.attn_scale:.6f}")
                self.current_epoch = epoch
            if c.save_every > 0 and self.step % c.save_every == 0:
                self.save_state(resume_path, {"min_bpb": min_bpb, "min_loss": min_loss, "bad_epochs": bad_epochs,
                                              "ring_paths": list(ring.paths)})
            if c.track == "tiny" and c.max_train_steps > 0 and self.step >= c.max_train_steps:
                print0(f"Reached max_train_steps={c.max_train_steps}")
                break
            if self.step == 1:
                gc.collect()
                gc.freeze()
                gc.disable()
        gc.enable()
        # ---------------------------------------------------------------- post-training averaging
        self.comm.barrier()          # every checkpoint rank 0 wrote is complete before any rank reads it
        comm = self.comm if world > 1 else None
        if c.track in self.LOGIT_AVG_TRACKS and c.logit_avg > 0:
            paths = ring.paths
            if c.eval_logit_avg:
                import glob
                paths = sorted(glob.glob(os.path.join(c.logit_avg_dir, "epoch_*.pt")))[-c.logit_avg:]
            if len(paths) >= 2:
                n = len(paths)
                print0(f"\n--- Evaluating logit avg ({n} checkpoints: {[os.path.basename(p) for p in paths]}) ---")
                if self.token_bytes is None:
                    self.token_bytes = default_token_bytes(self.device, c.model.vocab_size)
                steps = max(1, c.eval_tokens // (c.device_batch_size * c.model.sequence_len * world))
                self.model.eval()
                for label in (("equal", "weighted") if c.logit_avg_mode == "both" else (c.logit_avg_mode,)):
                    w = recency_weights(n, label)
                    print0(f"  [{label}] weights: {[f'{x:.3f}' for x in w]}")
                    with self.forward_context():
                        bpb, loss = evaluate_prob_avg(self.model, self.build_val_loader, paths, w, steps, self.token_bytes, comm)
                    print0(f"  [{label}] Val BPB: {bpb:.6f} | Val Loss: {loss:.6f}")
                    log.metrics({f"logit_avg_{label}/bpb": bpb, f"logit_avg_{label}/loss": loss})
                    if loss < min_loss:
                        min_loss, min_bpb = loss, bpb
                        print0(f"  ** New best! (logit avg {label} weights)")
        if c.track == "tiny":
            if self.ema is not None and self.ema.copy_into(self.model):
                val_bpb, val_loss = self.evaluate(max_iters)
                print0(f"EMA Val BPB: {val_bpb:.6f} | EMA Val Loss: {val_loss:.6f} | iters: {max_iters}")
                log.metrics({"step": self.step, "val/ema_bpb": val_bpb, "val/ema_loss": val_loss})
                if val_bpb < min_bpb:
                    min_bpb, min_loss = val_bpb, val_loss
            if len(ring.paths) >= 2:
                average_checkpoints_into(self.model, ring.paths, recency_weights(len(ring.paths)), comm, self.master)
                avg_bpb, avg_loss = self.evaluate(max_iters)
                print0(f"Ckpt avg Val BPB: {avg_bpb:.6f} | Val Loss: {avg_loss:.6f} | iters: {max_iters}")
                log.metrics({"ckpt_avg/bpb": avg_bpb, "ckpt_avg/loss": avg_loss})
                if avg_loss < min_loss:
                    min_loss, min_bpb = avg_loss, avg_bpb
            if self.master:
                torch.save({n: p.data.float().cpu() for n, p in self.model.named_parameters()}, os.path.join(log.run_dir, "model.pt"))
            self.comm.barrier()
        min_bpb, min_loss = self.post_training(log, (min_bpb, min_loss))
        peak = torch.cuda.max_memory_allocated() / 1024 / 1024 if self.device.type == "cuda" else 0.0
        final_train = self.smooth_loss / (1 - 0.9 ** self.step) if self.step > 0 else float("inf")
        print0(f"Peak memory: {peak:.2f} MiB")
        print0(f"Total training time: {total_time / 60:.2f}m")
        print0(f"Final train loss: {final_train:.6f}")
        print0(f"Min val BPB: {min_bpb:.6f}")
        print0(f"Min val Loss: {min_loss:.6f}")
        result = {"matrix_lr": c.matrix_lr, "weight_decay": c.weight_decay, "num_epochs": c.num_epochs,
                  "val_loss": val_loss, "best_val_loss": min_loss, "val_bpb": val_bpb, "best_val_bpb": min_bpb,
                  "final_train_loss": final_train, "steps": self.step, "training_time_s": total_time,
                  "peak_memory_mib": peak, "wandb_url": None}
        log.finish(result)
        return result
