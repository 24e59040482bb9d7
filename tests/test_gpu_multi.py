"""Multi-GPU checks of the peer-memory optimizer step (one child process per GPU): every variant of the fused step
(plain peer loads or in-switch multimem reads, bf16 or fp32 gradients on the wire, gradient pulls after the backward pass
or under it) must leave identical parameters on all ranks and follow the torch.distributed (NCCL) step. The model has
five layers, so the shape groups hold an odd number of matrices and the last rank owns fewer than the others."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# name -> (multimem, wire dtype, pulls under the backward pass)
VARIANTS = {
    "nccl": None,
    "p2p_fp32": (0, "fp32", False),
    "p2p_bf16": (0, "bf16", False),
    "p2p_bf16_overlap": (0, "bf16", True),
    "mm_bf16": (1, "bf16", False),
    "mm_bf16_overlap": (1, "bf16", True),
    "mm_fp32_overlap": (1, "fp32", True),
    "mm_bf16_pull_updates": (1, "bf16", False),      # update all-gather by peer loads instead of multicast stores
}
STEPS, ACCUM = 3, 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), SLOWRUN_PEER_WAIT_S="20")
    from slowrun_b200.config import track_defaults
    from slowrun_b200.parallel.comm import init_distributed, shutdown
    from slowrun_b200.parallel.fused import FusedComm
    info = init_distributed(timeout_s=120)
    cfg = track_defaults("limited")
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 5, 256, 2, 2, 256
    m.dropout, m.stoch_depth = 0.0, 0.0
    fused_comm = FusedComm()
    g = torch.Generator().manual_seed(7)
    data = torch.randint(0, 50257, (STEPS, ACCUM, world, 2, 257), generator=g)
    results = {}
    for name, var in VARIANTS.items():
        # A failure on one rank must not leave the others behind: every rank reports after every variant, and all stop
        # together (a rank never exits while the others still have kernels that read its memory in flight).
        err = None
        try:
            _run_variant(results, name, var, info, cfg, m, fused_comm, data, rank, world)
            torch.cuda.synchronize()
        except Exception:  # noqa: BLE001
            import traceback
            err = traceback.format_exc()
        flag = torch.tensor([1.0 if err else 0.0], device=info.device)
        torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MAX)
        if flag.item() > 0:
            results["error"] = err or "another rank failed"
            break
    torch.save(results, os.path.join(out, f"w{world}_r{rank}.pt"))
    torch.cuda.synchronize()
    torch.distributed.barrier()
    shutdown()


def _run_variant(results, name, var, info, cfg, m, fused_comm, data, rank, world):
    from slowrun_b200.models.gpt import build_model
    from slowrun_b200.optim.groups import build_param_groups
    from slowrun_b200.optim.muon_adamw import ShardedMuonAdamW
    from slowrun_b200.parallel.comm import TorchComm
    from slowrun_b200.ops import _lib
    if var is None:
        comm = TorchComm()
        model = build_model(m, info.device, seed=0, world_size=world)
        opt = ShardedMuonAdamW(model, build_param_groups(model, cfg), comm)
        overlap = False
    else:
        mm, wire, overlap = var
        os.environ["SLOWRUN_MULTIMEM"] = str(mm)
        os.environ["SLOWRUN_PUSH_UPDATES"] = "0" if name.endswith("pull_updates") else "1"
        model = build_model(m, info.device, seed=0, world_size=world, alloc=fused_comm.alloc)
        opt = ShardedMuonAdamW(model, build_param_groups(model, cfg), fused_comm, wire_dtype=wire)
        assert opt.fused
        opt.mode = "fused"
        some_group = next(iter(model.arena.groups.values()))
        has_mc = bool(fused_comm.multicast_ptr(some_group.G))
        if mm and not has_mc:
            results[name] = {"skipped": "no multicast mapping"}
            return
        assert has_mc == bool(mm)
        odd = [ga for ga in model.arena.groups.values() if ga.n % world]
        assert odd, "the test model must have a shape group whose matrix count is not a multiple of the world size"
    losses = []
    for s in range(STEPS):
        for a in range(ACCUM):
            b = data[s, a, rank].to(info.device)
            last = a == ACCUM - 1
            if overlap and last:
                assert opt.begin_backward_overlap()
            loss, _ = model(b[:, :-1], b[:, 1:])
            (loss / ACCUM).backward()
            if overlap and last:
                opt.finish_backward_overlap()
        opt.step()
        torch.cuda.synchronize()
        _lib.check_status()
        model.zero_grad_arena()
        losses.append(float(loss.detach()))
    if var is not None:
        assert fused_comm.check_guards() > 10        # no kernel of any rank wrote past the end of a symmetric buffer
    results[name] = {"losses": losses, "params": {n: p.detach().float().cpu() for n, p in model.named_parameters()}}


def _rel(a, b):
    num = sum((a[n] - b[n]).pow(2).sum() for n in a)
    den = sum(a[n].pow(2).sum() for n in a)
    return (num / den).sqrt().item()


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world", [2, 4])
def test_fused_peer_memory_step_variants_match_nccl_path(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = str(tmp_path)
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    res = [torch.load(os.path.join(out, f"w{world}_r{r}.pt")) for r in range(world)]
    for r in range(world):
        assert "error" not in res[r], f"rank {r}:\n{res[r]['error']}"
    ref = res[0]["nccl"]
    ran = []
    for name in VARIANTS:
        if name == "nccl" or "skipped" in res[0][name]:
            continue
        ran.append(name)
        r0 = res[0][name]
        for r in range(1, world):
            for n in r0["params"]:
                assert torch.equal(r0["params"][n], res[r][name]["params"][n]), f"{name}: replicas diverged in {n}"
        assert abs(ref["losses"][0] - r0["losses"][0]) < 1e-3, name
        assert _rel(ref["params"], r0["params"]) < 2e-2, (name, _rel(ref["params"], r0["params"]))
        assert abs(ref["losses"][-1] - r0["losses"][-1]) < 5e-2, name      # same trajectory
    assert "p2p_fp32" in ran and "p2p_bf16_overlap" in ran
    # pulling under the backward pass changes the launch grouping, not the arithmetic
    for a, b in (("p2p_bf16", "p2p_bf16_overlap"), ("mm_bf16", "mm_bf16_overlap")):
        if a in ran and b in ran:
            # (atomics order the sums differently from run to run and Newton-Schulz magnifies that: a few 1e-3 is the
            # run-to-run spread of one and the same variant)
            assert _rel(res[0][a]["params"], res[0][b]["params"]) < 8e-3, (a, b, _rel(res[0][a]["params"], res[0][b]["params"]))
    # the bf16 wire costs at most bf16 rounding of the summed gradient
    assert _rel(res[0]["p2p_fp32"]["params"], res[0]["p2p_bf16"]["params"]) < 1e-2


def _ddp_worker(rank, world, port, out):
    """Unlimited-track gradient path on GPUs: bucketed NCCL all-reduce issued from the backward pass against the plain
    all-reduce after it, and one full trainer step of a two-rank node."""
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from slowrun_b200.config import track_defaults
    from slowrun_b200.models.gpt import build_model
    from slowrun_b200.parallel.comm import TorchComm, init_distributed, shutdown
    from slowrun_b200.train.unlimited import OverlappedAllReduce, allreduce_gradients
    from slowrun_b200.ops import _lib
    info = init_distributed(timeout_s=120)
    res = {}
    try:
        cfg = track_defaults("unlimited")
        m = cfg.model
        m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 4, 256, 2, 2, 256
        m.dropout = 0.0
        model = build_model(m, info.device, seed=0)
        model.set_dupe_layers(2, 3, 1)
        comm = TorchComm()
        g = torch.Generator().manual_seed(10 + rank)
        idx = torch.randint(0, 50257, (2, 257), generator=g).to(info.device)
        grads = {}
        for mode in ("plain", "overlapped"):
            model.zero_grad_arena()
            red = OverlappedAllReduce(model, comm) if mode == "overlapped" else None
            if red is not None:
                red.arm()
            loss, _ = model(idx[:, :-1], idx[:, 1:])
            loss.backward()
            if red is not None:
                early = len(red.handles)
                red.finish()
            else:
                allreduce_gradients(model, comm)
            torch.cuda.synchronize()
            _lib.check_status()
            grads[mode] = {n: (model.arena.head_grad if n == "lm_head.weight" else p.grad).float().cpu().clone()
                           for n, p in model.named_parameters()}
        res = {"grads": grads, "early": early}
    except Exception:  # noqa: BLE001
        import traceback
        res = {"error": traceback.format_exc()}
    torch.save(res, os.path.join(out, f"ddp_r{rank}.pt"))
    torch.cuda.synchronize()
    torch.distributed.barrier()
    shutdown()


@pytest.mark.timeout(600)
def test_bucketed_allreduce_under_backward_matches_plain_allreduce_on_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mp.spawn(_ddp_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    r0, r1 = (torch.load(tmp_path / f"ddp_r{r}.pt") for r in (0, 1))
    assert "error" not in r0, r0.get("error")
    assert "error" not in r1, r1.get("error")
    worst = 0.0
    for n in r0["grads"]["plain"]:
        a, b = r0["grads"]["plain"][n], r0["grads"]["overlapped"][n]
        assert torch.equal(b, r1["grads"]["overlapped"][n]), n            # both ranks hold the same reduced gradient
        worst = max(worst, ((a - b).norm() / a.norm().clamp_min(1e-20)).item())
    # the two backward passes accumulate weight gradients through split-K reductions whose order is not fixed
    assert worst < 1e-3, worst
    assert r0["early"] > 0
