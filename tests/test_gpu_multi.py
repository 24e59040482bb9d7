"""Two-GPU checks of the peer-memory collectives: the fused optimizer step must produce the same parameters as the
NCCL path and as a single-GPU run on the concatenated batch. Runs as child processes, one per GPU, with NVLS off."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, out):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    from slowrun_b200.config import track_defaults
    from slowrun_b200.models.gpt import build_model
    from slowrun_b200.optim.groups import build_param_groups
    from slowrun_b200.optim.muon_adamw import ShardedMuonAdamW
    from slowrun_b200.parallel.comm import TorchComm, init_distributed, shutdown
    from slowrun_b200.ops import _lib
    info = init_distributed(timeout_s=120)
    cfg = track_defaults("limited")
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 4, 256, 2, 2, 256
    m.dropout, m.stoch_depth = 0.0, 0.0
    if mode == "fused":
        from slowrun_b200.parallel.fused import FusedComm
        comm = FusedComm()
        model = build_model(m, info.device, seed=0, world_size=world, alloc=comm.alloc)
    else:
        comm = TorchComm()
        model = build_model(m, info.device, seed=0, world_size=world)
    opt = ShardedMuonAdamW(model, build_param_groups(model, cfg), comm)
    assert opt.fused == (mode == "fused")
    g = torch.Generator().manual_seed(7)
    data = torch.randint(0, 50257, (3, world, 2, 257), generator=g)
    losses = []
    for s in range(3):
        b = data[s, rank].to(info.device)
        loss, _ = model(b[:, :-1], b[:, 1:])
        loss.backward()
        opt.step()
        model.zero_grad_arena()
        losses.append(float(loss.detach()))
    torch.cuda.synchronize()
    _lib.check_status()
    torch.save({"losses": losses, "params": {n: p.detach().float().cpu() for n, p in model.named_parameters()}},
               os.path.join(out, f"{mode}_r{rank}.pt"))
    torch.distributed.barrier()
    shutdown()


@pytest.mark.timeout(600)
def test_fused_peer_memory_step_matches_nccl_path(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    out = str(tmp_path)
    for mode in ("nccl", "fused"):
        mp.spawn(_worker, args=(2, _free_port(), mode, out), nprocs=2, join=True)
    a0 = torch.load(os.path.join(out, "nccl_r0.pt"))
    f0 = torch.load(os.path.join(out, "fused_r0.pt"))
    f1 = torch.load(os.path.join(out, "fused_r1.pt"))
    for n in f0["params"]:
        assert torch.equal(f0["params"][n], f1["params"][n]), f"replicas diverged: {n}"
    assert abs(a0["losses"][0] - f0["losses"][0]) < 1e-3
    num = sum((a0["params"][n] - f0["params"][n]).pow(2).sum() for n in a0["params"])
    den = sum(a0["params"][n].pow(2).sum() for n in a0["params"])
    assert (num / den).sqrt().item() < 2e-2, (num / den).sqrt().item()
    assert abs(a0["losses"][-1] - f0["losses"][-1]) < 5e-2      # both paths follow the same trajectory
