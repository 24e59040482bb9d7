"""Run directory, stdout tee, metrics sinks and result.json.

Mirrors the reference's observability (train.py:155-179, 981-1007, 1301-1336): `runs/<name>/` with a copy of the
entry script, `terminal.log` teeing stdout/stderr on rank 0, wandb project "slowrun" (here strictly optional and
off by default — the reference calls wandb.init unconditionally), plus a JSONL metrics file that needs no service.
"""
from __future__ import annotations

import json
import os
import shutil
import sys
import time

import torch

from ..parallel.comm import print0

# bf16 dense peak FLOP/s used for the MFU print. The reference knows H100/A100/4090 and prints 0 elsewhere
# (train.py:966-972); B200's nominal dense bf16 rate is added here.
PEAK_FLOPS = {"b200": 2.25e15, "h100": 989e12, "a100": 312e12, "4090": 165.2e12}


class TeeStream:
    def __init__(self, *streams):
        self.streams = streams
        self.encoding = getattr(streams[0], "encoding", "utf-8")

    def write(self, data):
        for s in self.streams:
            s.write(data)
        return len(data)

    def flush(self):
        for s in self.streams:
            s.flush()

    def isatty(self):
        return any(getattr(s, "isatty", lambda: False)() for s in self.streams)

    def fileno(self):
        return self.streams[0].fileno()


class DummyWandb:
    def __init__(self):
        self.summary = {}

    def log(self, *a, **kw):
        pass

    def finish(self):
        pass


def gpu_peak_flops() -> float:
    if not torch.cuda.is_available():
        return float("inf")
    name = torch.cuda.get_device_name(0).lower()
    for key, val in PEAK_FLOPS.items():
        if key in name:
            return val
    return float("inf")


class RunLogger:
    def __init__(self, cfg, info, quiet=False, script_path=None):
        self.cfg, self.info = cfg, info
        self.master = info.rank == 0
        name = cfg.run_name or time.strftime("%Y%m%d_%H%M%S")
        if info.world_size > 1 and torch.distributed.is_initialized():
            shared = [name]
            torch.distributed.broadcast_object_list(shared, src=0)
            name = shared[0]
        self.run_name = name
        self.run_dir = os.path.join(cfg.runs_dir, name)
        self.peak_flops = gpu_peak_flops()
        self._orig = (sys.stdout, sys.stderr)
        self._log_f = None
        self._jsonl = None
        self.wandb = DummyWandb()
        if self.master and not quiet:
            os.makedirs(os.path.join(self.run_dir, "checkpoints"), exist_ok=True)
            script = script_path or (sys.argv[0] if sys.argv and os.path.isfile(sys.argv[0]) else None)
            if script:
                try:
                    shutil.copy2(script, os.path.join(self.run_dir, os.path.basename(script)))
                except OSError:
                    pass
            self._log_f = open(os.path.join(self.run_dir, "terminal.log"), "a", encoding="utf-8", buffering=1)
            sys.stdout = TeeStream(sys.stdout, self._log_f)
            sys.stderr = TeeStream(sys.stderr, self._log_f)
            self._jsonl = open(cfg.log_jsonl or os.path.join(self.run_dir, "metrics.jsonl"), "a", buffering=1)
            if cfg.wandb:
                try:
                    import wandb
                    kw = {"project": "slowrun", "name": name, "dir": os.path.join(self.run_dir, "wandb")}
                    if cfg.wandb_group:
                        kw["group"] = cfg.wandb_group
                    os.makedirs(kw["dir"], exist_ok=True)
                    self.wandb = wandb.init(**kw)
                except Exception as e:  # noqa: BLE001
                    print0(f"wandb unavailable ({e}); continuing with JSONL metrics only")
        elif self.master:
            os.makedirs(self.run_dir, exist_ok=True)

    def hyperparameters(self, cfg, model, flops_per_token):
        m = cfg.model
        lrs = cfg.lrs
        print0("--- Hyperparameters ---")
        print0(f"  track={cfg.track}")
        print0(f"  n_layer={m.n_layer}, n_embd={m.n_embd}, n_head={m.n_head}, head_dim={m.head_dim}")
        print0(f"  seq_len={m.sequence_len}, window_pattern={m.window_pattern}")
        print0(f"  stoch_depth={m.stoch_depth}")
        print0(f"  total_batch_size={cfg.total_batch_size}, device_batch_size={cfg.device_batch_size}")
        print0(f"  matrix_lr={lrs['matrix']}, scalar_lr={lrs['scalar']}, embedding_lr={lrs['embedding']}, unembedding_lr={lrs['unembedding']}")
        print0(f"  weight_decay={cfg.weight_decay}, adam_betas={tuple(cfg.adam_betas)}")
        print0(f"  warmup_ratio={cfg.warmup_ratio}, warmdown_ratio={cfg.warmdown_ratio}, final_lr_frac={cfg.final_lr_frac}")
        print0(f"  num_epochs={cfg.num_epochs}, patience={cfg.patience}")
        print0(f"  dropout={m.dropout}, doc_shuffle={not cfg.no_doc_shuffle}")
        print0(f"  run={self.run_name}")
        print0(f"  run_dir={self.run_dir}")
        if m.use_iha:
            print0(f"  iha=True, iha_lr={cfg.iha_lr}")
        print0("-----------------------")
        total = sum(p.numel() for p in model.parameters())
        tr = sum(p.numel() for p in model.transformer.h.parameters())
        ve = sum(p.numel() for p in model.ve_projs.parameters())
        lm = model.lm_head.weight.numel()
        print0(f"Parameters: {total:,} (transformer: {tr:,}, value_embeds: {ve:,}, lm_head: {lm:,}, other: {total - tr - ve - lm:,})")
        print0(f"FLOPs per token: {flops_per_token:e}")

    def metrics(self, d: dict):
        if self._jsonl is not None:
            self._jsonl.write(json.dumps(d) + "\n")
        self.wandb.log(d)

    def finish(self, result: dict):
        out = self.cfg.save_result or (os.path.join(self.run_dir, "result.json") if self.cfg.track in ("limited", "tiny") else "")
        if self.master and out:
            os.makedirs(os.path.dirname(os.path.abspath(out)), exist_ok=True)
            with open(out, "w") as f:
                json.dump(result, f, indent=2)
            print0(f"Result saved to {out}")
        self.wandb.finish()
        if self._jsonl is not None:
            self._jsonl.close()
        if self._log_f is not None:
            sys.stdout.flush()
            sys.stderr.flush()
            sys.stdout, sys.stderr = self._orig
            self._log_f.close()
