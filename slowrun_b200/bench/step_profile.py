"""Where one micro-step (forward + loss + backward of one device batch) and one optimizer step spend their GPU time.

    python -m slowrun_b200.bench.step_profile [--track limited|tiny] [--size 2.7b] [--batch N] [--top 40]

Runs the limited-track (or tiny-track) model eagerly (no CUDA graph, so kernels keep their names), times a micro-step and an optimizer
step with CUDA events, then records one of each with the CUPTI activity tracer (`torch.profiler`, device activities
only) and prints per-kernel totals: name, launches, total µs, share. The times inside the traced pass are for shares
only; the event-timed figures printed first are the ones to quote.
"""
from __future__ import annotations

import argparse
import collections
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def kernel_table(fn, top):
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        fn()
        torch.cuda.synchronize()
    tot = collections.defaultdict(lambda: [0, 0.0])
    for ev in prof.events():
        if ev.device_type == torch.autograd.DeviceType.CUDA:
            t = tot[ev.name]
            t[0] += 1
            t[1] += ev.device_time
    total = sum(v[1] for v in tot.values())
    rows = sorted(tot.items(), key=lambda kv: -kv[1][1])[:top]
    lines = [f"{'kernel':90s} {'n':>5s} {'us':>10s} {'share':>6s}"]
    for name, (n, us) in rows:
        lines.append(f"{name[:90]:90s} {n:5d} {us:10.0f} {100 * us / total:5.1f}%")
    lines.append(f"{'total':90s} {'':5s} {total:10.0f}")
    return "\n".join(lines)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", default="2.7b", choices=["2.7b", "default"])
    ap.add_argument("--track", default="limited", choices=["limited", "tiny"])
    ap.add_argument("--batch", type=int, default=0, help="sequences per micro-batch (default: 4 limited, 32 tiny)")
    ap.add_argument("--top", type=int, default=40)
    a = ap.parse_args()
    sys.path.insert(0, ROOT)
    from slowrun_b200.config import track_defaults
    from slowrun_b200.models.gpt import build_model
    from slowrun_b200.optim.groups import build_param_groups
    from slowrun_b200.optim.muon_adamw import ShardedMuonAdamW
    from slowrun_b200.parallel.comm import TorchComm

    cfg = track_defaults(a.track)
    tiny = a.track == "tiny"
    a.batch = a.batch or (32 if tiny else 4)
    if a.size == "2.7b" and not tiny:
        cfg.model.n_embd, cfg.model.n_head, cfg.model.n_kv_head = 2560, 20, 20
    model = build_model(cfg.model, "cuda", seed=0)
    opt = ShardedMuonAdamW(model, build_param_groups(model, cfg), TorchComm())
    T = cfg.model.sequence_len
    idx = torch.randint(0, 50257, (a.batch, T), device="cuda")
    tgt = torch.randint(0, 50257, (a.batch, T), device="cuda")

    mtp_w = torch.tensor([1.0, 0.5, 0.25], device="cuda") if (tiny and cfg.model.fused_mtp) else None

    def micro():
        if tiny:
            loss = model(idx, tgt, num_iterations=cfg.model.num_iterations, mtp_weights=mtp_w)
        else:
            loss, _ = model(idx, tgt)
        loss.backward()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    for _ in range(3):
        micro()
    opt.step()
    model.zero_grad_arena()
    torch.cuda.synchronize()
    print(f"micro-step {timed(micro, 5):.2f} ms   optimizer step {timed(opt.step, 2):.2f} ms   (CUDA events, eager)")
    print("\n== micro-step kernels\n" + kernel_table(micro, a.top))
    print("\n== optimizer-step kernels\n" + kernel_table(opt.step, a.top))


if __name__ == "__main__":
    main()
