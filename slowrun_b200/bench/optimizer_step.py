"""Distributed Muon/AdamW optimizer step of the 2.7 B limited-track model: peer-memory fused path against the
NCCL path, on N ranks of one node.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m slowrun_b200.bench.optimizer_step [--size 2.7b] [--iters 5]

Both paths run the same update (`ShardedMuonAdamW.step`): the NCCL one as reduce-scatter -> Muon on the owned chunk ->
all-gather -> apply (the reference's structure, train.py:656-760), the fused one with the gradients pulled from the
peers inside the Muon prologue and the bf16 updates pulled inside the apply kernel (csrc/comm_fused.cu). Gradients
are random and fixed; every iteration is one full step. Times are CUDA events, max over ranks. Rank 0 prints one
JSON line with both times, the bytes each rank must receive over NVLink, the Newton-Schulz FLOPs per rank, and the
roofline = max(FLOPs / measured bf16 peak, bytes / 770 GB/s) with achieved = roofline / time.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
LINK_GBS = 770.0      # measured peer copy bandwidth per direction per GPU on this pool


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", default="2.7b", choices=["2.7b", "1.4b"])
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    sys.path.insert(0, ROOT)
    from slowrun_b200.config import track_defaults
    from slowrun_b200.models.gpt import build_model
    from slowrun_b200.optim.groups import build_param_groups
    from slowrun_b200.optim.muon_adamw import ShardedMuonAdamW
    from slowrun_b200.parallel.comm import TorchComm, init_distributed
    from slowrun_b200.parallel.fused import FusedComm
    from slowrun_b200.ops import _lib

    info = init_distributed()
    W, rank, dev = info.world_size, info.rank, info.device
    cfg = track_defaults("limited")
    if a.size == "2.7b":
        cfg.model.n_embd, cfg.model.n_head, cfg.model.n_kv_head = 2560, 20, 20
    fused = FusedComm() if W > 1 else None
    model = build_model(cfg.model, dev, seed=0, world_size=W, alloc=fused.alloc if fused else None)
    groups = build_param_groups(model, cfg)
    opts = {"nccl": ShardedMuonAdamW(model, groups, TorchComm())}
    if fused is not None:
        opts["fused"] = ShardedMuonAdamW(model, groups, fused, wire_dtype="bf16")
        opts["fused_overlap"] = opts["fused"]
        opts["fused_fp32_wire"] = ShardedMuonAdamW(model, groups, fused, wire_dtype="fp32")
    gen = torch.Generator(device=dev).manual_seed(1 + rank)
    for ga in model.arena.groups.values():
        ga.G.normal_(0, 0.02, generator=gen)
    for p in model.parameters():
        if p.grad is not None and p.grad.dtype == torch.float32 and p.grad.numel() < (1 << 24):
            p.grad.normal_(0, 0.02, generator=gen)
    if model.arena.head_grad is not None:
        model.arena.head_grad.normal_(0, 0.02, generator=gen)

    def timed(opt):
        for _ in range(2):
            opt.step()
        torch.cuda.synchronize()
        if W > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            opt.step()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
        if W > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    res = {}
    for k, o in opts.items():
        if k != "nccl":
            o.mode = "fused_two_streams" if k == "fused_overlap" else "fused"   # fused_fp32_wire: one stream, fp32 pulls
        res[k] = timed(o)
    if fused is not None:
        o = opts["fused"]
        o.mode, o.overlap = "auto", "auto"   # measuring steps, then the fastest formulation
        o.__dict__.pop("_tune", None)
        while o.tuning_steps_left > 0:
            o.step()
        res["auto"] = timed(o)
    _lib.check_status()
    phases = None
    if "fused" in opts:
        o = opts["fused"]
        chosen = getattr(o, "tuned", None)
        o.mode = "fused"
        o.trace_phases = True
        o.step()
        phases = {k: round(v, 3) for k, v in o.phase_report().items()}
        o.trace_phases = False
        o.tuned = chosen
    # traffic and FLOPs per rank
    g_bytes = sum(ga.G.numel() * 4 for ga in model.arena.groups.values())            # fp32 stacked gradients
    u_bytes = g_bytes // 2                                                            # bf16 updates
    rs_in = (g_bytes // 2 // W) * (W - 1) if W > 1 else 0                             # own chunk from each peer, bf16 wire
    ag_in = (u_bytes // W) * (W - 1) if W > 1 else 0
    ns_flops = 0.0
    for ga in model.arena.groups.values():
        r, c = ga.shape
        gdim, o = min(r, c), max(r, c)
        ns_flops += 5 * ga.chunk * (4.0 * gdim * gdim * o + 2.0 * gdim ** 3)   # the reference's 15 full bmm's
    try:
        peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]
        src = "measured"
    except Exception:  # noqa: BLE001
        peak, src = 1590.0, "fallback"
    t_compute = ns_flops / (peak * 1e9)          # ms
    t_link = (rs_in + ag_in) / (LINK_GBS * 1e6)  # ms
    roof = max(t_compute, t_link)
    if rank == 0:
        out = {"what": "optimizer_step", "size": a.size, "n_gpus": W, "ms": res,
               "nvlink_bytes_in_per_rank": {"grad_pull": rs_in, "update_pull": ag_in},
               "ns_tflop_per_rank": ns_flops / 1e12, "roofline_ms": {"compute": t_compute, "link": t_link, "peaks": src},
               "frac_of_roofline": {k: roof / v for k, v in res.items()}, "fused_phases_ms_rank0": phases,
               "auto_choice": getattr(opts.get("fused"), "tuned", None) if fused is not None else None,
               "nvls_multimem_pull": bool(fused is not None and fused.multicast_ptr(next(iter(model.arena.groups.values())).G))}
        print(json.dumps(out))
    if W > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
