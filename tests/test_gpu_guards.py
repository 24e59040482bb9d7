"""GPU runs of the memory-checker and race-detector stand-ins: every buffer the op layer allocates during a training
step (ragged sequence length, ragged vocabulary tile, both tracks' block variants) carries red zones that must be intact
afterwards, and repeated runs from the same inputs must agree (bit for bit for the forward pass; gradients that are
accumulated with floating-point atomics within a tolerance)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _model(track, T):
    from slowrun_b200.config import track_defaults
    from slowrun_b200.models.gpt import build_model
    cfg = track_defaults(track)
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 3, 256, 2, 2, T
    m.dropout, m.stoch_depth = 0.0, 0.0
    return build_model(m, torch.device("cuda"), seed=0), cfg


@pytest.mark.parametrize("track,T", [("limited", 200), ("limited", 384), ("tiny", 328)])
def test_no_kernel_writes_outside_its_buffers(track, T):
    from slowrun_b200.ops import _lib
    from slowrun_b200.utils.debug import RedZones
    model, cfg = _model(track, T)
    idx = torch.randint(0, 50257, (3, T + 1), device="cuda")
    with RedZones() as zones:
        for _ in range(2):
            out = model(idx[:, :-1], idx[:, 1:])
            loss = out[0] if isinstance(out, tuple) else out
            loss.backward()
        torch.cuda.synchronize()
        _lib.check_status()
        assert zones.check() > 50
    assert torch.isfinite(loss).item()


def test_forward_is_bit_reproducible_and_gradients_agree():
    from slowrun_b200.utils.debug import repeat_check
    model, cfg = _model("limited", 256)
    idx = torch.randint(0, 50257, (4, 257), device="cuda")

    def forward():
        with torch.no_grad():
            loss, _ = model(idx[:, :-1], idx[:, 1:])
        return loss

    repeat_check(forward, times=4)

    def grads():
        model.zero_grad_arena()
        loss, _ = model(idx[:, :-1], idx[:, 1:])
        loss.backward()
        torch.cuda.synchronize()
        return [ga.G for ga in model.arena.groups.values()]

    # weight gradients leave the GEMM through split-K vector reductions whose order is not fixed
    repeat_check(grads, times=3, atol=2e-3)


def test_debug_check_build_runs_a_step_clean():
    """The library variant with the in-kernel index/alignment checks compiled in (SLOWRUN_DEBUG_CHECKS=1) runs a
    ragged-shape training step without a single check firing."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import torch\n"
        "from slowrun_b200.ops import _lib\n"
        "assert _lib.library_path().endswith('_kernels_debug.so')\n"
        "from slowrun_b200.config import track_defaults\n"
        "from slowrun_b200.models.gpt import build_model\n"
        "from slowrun_b200.optim.groups import build_param_groups\n"
        "from slowrun_b200.optim.muon_adamw import ShardedMuonAdamW\n"
        "from slowrun_b200.parallel.comm import TorchComm\n"
        "cfg = track_defaults('limited'); m = cfg.model\n"
        "m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 3, 256, 2, 2, 200\n"
        "model = build_model(m, 'cuda:0', seed=0)\n"
        "opt = ShardedMuonAdamW(model, build_param_groups(model, cfg), TorchComm())\n"
        "idx = torch.randint(0, 50257, (3, 201), device='cuda:0')\n"
        "for _ in range(2):\n"
        "    loss, _ = model(idx[:, :-1], idx[:, 1:]); loss.backward(); opt.step(); model.zero_grad_arena()\n"
        "torch.cuda.synchronize(); _lib.check_status(); print('debug-ok', float(loss))\n")
    env = dict(os.environ, SLOWRUN_DEBUG_CHECKS="1")
    res = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "debug-ok" in res.stdout, res.stdout + res.stderr
