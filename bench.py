"""Headline benchmark: training tokens/s of the limited-track GPT at the "2.7 B" size (30 layers, d_model 2560,
20 heads of 128, SwiGLU 6912, IHA, MTP block, dropout 0.1, stochastic depth 0.05, vocab 50257 -> 50304, seq 2048,
524 288 tokens per optimizer step) on N GPUs of one node, bf16, synthetic Zipf(1.1) tokens, random-init weights.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...     # the unmodified reference script through baseline/ref_runner.py
    python bench.py --track tiny ...         # same measurement for the tiny track (16 layers, d_model 1024, 8 heads,
                                             # recurrence, XSA, fp8 shared-head multi-token loss, device batch 32)

One "step" is one optimizer step of the reference's loop (train.py:1156-1187): total_batch/(B*T*N) micro-batches of
forward+backward with local gradient accumulation, then the sharded Muon/AdamW step with all its communication.
Rank 0 prints ONE JSON line. `value` is device-timed (CUDA events around exactly K steps, max over ranks); `e2e` is
a second timed region through the public API (`Trainer.train_step()`), host-clocked, where every micro-batch is
copied from pinned host memory and the step's loss is read back to the host.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SIZES = {
    # name: (n_layer, n_embd, n_head)
    "2.7b": (30, 2560, 20),
    "1.4b": (30, 1792, 14),
    "smoke": (4, 256, 2),
    "tiny": (16, 1024, 8),
}


class ClockSampler:
    """Samples SM clock / throttle reasons with nvidia-smi while the timed region runs (read-only queries)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="clocks_", suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:  # noqa: BLE001
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        try:
            rows = [r.strip().split(",") for r in open(self.path) if r.strip()]
            os.remove(self.path)
        except Exception:  # noqa: BLE001
            return out
        sm, mx, reasons = [], [], set()
        for r in rows:
            r = [x.strip() for x in r]
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            sm.sort()
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
    ids = [v.strip() for v in vis.split(",") if v.strip()]
    if local_rank < len(ids) and ids[local_rank].isdigit():
        return int(ids[local_rank])
    return local_rank


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    p.add_argument("--track", type=str, default="limited", choices=["limited", "tiny"])
    p.add_argument("--size", type=str, default=None, choices=list(SIZES))
    p.add_argument("--device-batch-size", type=int, default=None)
    p.add_argument("--total-batch-size", type=int, default=524288)
    p.add_argument("--comm", type=str, default="auto", choices=["auto", "fused", "nccl"])
    p.add_argument("--no-e2e", action="store_true")
    a = p.parse_args()
    if a.size is None:
        a.size = "tiny" if a.track == "tiny" else "2.7b"
    if a.device_batch_size is None:
        a.device_batch_size = 32 if a.track == "tiny" else 4
    return a


def ensure_corpus(args, rank, world, barrier):
    """Synthetic Zipf corpus in the reference's format, written once per job by rank 0."""
    from slowrun_b200.data.synthetic import write_synthetic_corpus
    need = (args.warmup + 2 * args.steps + 3 + 12) * args.total_batch_size
    d = os.path.join(tempfile.gettempdir(), f"slowrun_synth_{need}")
    if rank == 0 and not os.path.exists(os.path.join(d, "fineweb_train.pt")):
        write_synthetic_corpus(d + ".tmp", train_tokens=int(need * 1.02) + 2049 * 64, val_tokens=1_100_000)
        os.replace(d + ".tmp", d)
    barrier()
    return d


def result_line(args, world, tok_per_s, ms_per_step, e2e, clocks, launches, extra):
    n_layer, n_embd, n_head = SIZES[args.size]
    line = {
        "metric": "train_tokens_per_s", "value": tok_per_s, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic Zipf(s=1.1) tokens over 50257 ids in the reference .pt format; random-init weights",
        "config": {"model": (f"tiny-track GPT: n_layer={n_layer} n_embd={n_embd} n_head={n_head} head_dim=128 swiglu XSA "
                             f"key-offset 2x-recurrence fp8 shared-head MTP dropout=0.1 vocab=50257" if args.track == "tiny" else
                             f"limited-track GPT {args.size}: n_layer={n_layer} n_embd={n_embd} n_head={n_head} head_dim=128 "
                             f"swiglu IHA MTP dropout=0.1 stoch_depth=0.05 vocab=50257"),
                   "global_batch": args.total_batch_size, "seq_len": 2048, "device_batch_size": args.device_batch_size,
                   "parallelism": f"dp{world} (optimizer-sharded)", "tokens_per_step": args.total_batch_size,
                   "l2": "working set (parameters + activations) is far larger than the 126 MB L2; no flush needed"},
        "clocks": clocks, "gpu_launches": launches,
    }
    if e2e is not None:
        line["e2e"] = e2e
    line.update(extra)
    return line


def run_ours(args):
    import torch
    from slowrun_b200.config import track_defaults
    from slowrun_b200.ops import _lib
    from slowrun_b200.parallel.comm import init_distributed, shutdown
    from slowrun_b200.train.trainer import Trainer
    import torch.distributed as dist

    info = init_distributed()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    world, rank = info.world_size, info.rank
    if world != args.gpus and rank == 0:
        print(f"[bench] note: --gpus {args.gpus} but WORLD_SIZE={world}; using {world}", file=sys.stderr)

    def barrier():
        if world > 1:
            dist.barrier()

    data_dir = ensure_corpus(args, rank, world, barrier)
    cfg = track_defaults(args.track)
    cfg.model.n_layer, cfg.model.n_embd, cfg.model.n_head = SIZES[args.size]
    cfg.model.n_kv_head = cfg.model.n_head
    cfg.device_batch_size = args.device_batch_size
    cfg.total_batch_size = args.total_batch_size
    cfg.input_bin = os.path.join(data_dir, "fineweb_train.pt")
    cfg.input_val_bin = os.path.join(data_dir, "fineweb_val.pt")
    cfg.comm = args.comm
    trainer = Trainer(cfg, info, quiet=True)
    tokens_per_step = cfg.total_batch_size

    def sync():
        barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        trainer.train_step(sync=True)
    # On more than one GPU the optimizer measures its step formulations during its first steps and then keeps the
    # fastest; the timed region below must see the kept one, so warm up until that choice is made.
    while getattr(trainer.optimizer, "tuning_steps_left", 0) > 0:
        trainer.train_step(sync=True)
    # ---------------------------------------------------------------- device-timed region
    sampler = ClockSampler(physical_gpu_index(info.local_rank))
    sync()
    if rank == 0:
        sampler.start()
    l0 = _lib.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        trainer.train_step(sync=False)
    e1.record()
    sync()
    launches = _lib.launch_count - l0
    _lib.check_status(info.device)
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=info.device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms) / args.steps
    tok_per_s = tokens_per_step / (ms_per_step / 1000.0)
    # ---------------------------------------------------------------- end-to-end region (public API, host clock)
    e2e = None
    if not args.no_e2e:
        sync()
        t0 = time.perf_counter()
        last = None
        for _ in range(args.steps):
            last = trainer.train_step(sync=True)["loss"]     # pinned-host -> device copies inside; loss read back
        torch.cuda.synchronize()
        dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=info.device)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        e2e = {"value": tokens_per_step * args.steps / float(dt), "unit": "tokens/s",
               "h2d_bytes_per_step": trainer.h2d_bytes_per_step, "d2h_bytes_per_step": trainer.d2h_bytes_per_step,
               "last_loss": last}
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        extra = {"impl": "ours", "comm": trainer.comm.name, "grad_accum": trainer.grad_accum,
                 "flops_per_token": trainer.flops_per_token,
                 "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30}
        print(json.dumps(result_line(args, world, tok_per_s, ms_per_step, e2e, clocks, launches, extra)), flush=True)
    barrier()
    shutdown()


def run_reference(args):
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import ref_runner
        if not ref_runner.reference_available():
            raise RuntimeError("baseline/_ref/train.py not present (the reference has no setup.py/pyproject to install)")
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
        rank = int(os.environ.get("RANK", 0))
        world = int(os.environ.get("WORLD_SIZE", 1))
        data_dir = os.path.join(tempfile.gettempdir(), f"slowrun_ref_synth_{args.total_batch_size}_{args.warmup + args.steps}")
        if rank == 0 and not os.path.exists(os.path.join(data_dir, "fineweb_train.pt")):
            from slowrun_b200.data.synthetic import write_synthetic_corpus
            need = (args.warmup + args.steps + 3) * args.total_batch_size
            write_synthetic_corpus(data_dir + ".tmp", train_tokens=int(need * 1.02) + 2049 * 64, val_tokens=1_100_000)
            os.replace(data_dir + ".tmp", data_dir)
        else:
            t0 = time.time()
            while not os.path.exists(os.path.join(data_dir, "fineweb_train.pt")) and time.time() - t0 < 300:
                time.sleep(0.5)
        n_layer, n_embd, n_head = SIZES[args.size]
        extra = ["--n_layer", str(n_layer), "--n_embd", str(n_embd), "--n_head", str(n_head),
                 "--device-batch-size", str(args.device_batch_size), "--total-batch-size", str(args.total_batch_size),
                 "--run-name", f"bench_ref_{args.track}_{os.getpid() if world == 1 else 'dist'}"]
        sampler = ClockSampler(0)
        if rank == 0:
            sampler.start()
        work = os.path.join(tempfile.gettempdir(), "slowrun_ref_work")
        res = ref_runner.run(args.track, args.steps, args.warmup, extra, data_dir, work)
        clocks = sampler.stop() if rank == 0 else None
        if rank == 0:
            ms_per_step = res["device_ms"] / args.steps
            line = result_line(args, world, args.total_batch_size / (ms_per_step / 1000.0), ms_per_step,
                               {"value": args.total_batch_size * args.steps / (res["host_ms"] / 1000.0), "unit": "tokens/s",
                                "h2d_bytes_per_step": args.total_batch_size // 2048 * 2049 * 8 // world,
                                "d2h_bytes_per_step": 4},
                               clocks, None, {"impl": "reference", "attn_backend": res["attn_backend"], "note": res.get("note")})
            print(json.dumps(line), flush=True)
    except BaseException as e:  # noqa: BLE001 - the contract is one JSON line and exit code 0
        if int(os.environ.get("RANK", 0)) == 0:
            sys.stdout = sys.__stdout__
            why = f"{type(e).__name__}: {str(e).splitlines()[0] if str(e) else ''}"[:300]
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    sys.exit(0)


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
