"""CPU fp32 parity of the model, loss and gradients against the reference's GPT (limited track)."""
import pytest
import torch

from slowrun_b200.config import ModelConfig
from slowrun_b200.models.gpt import GPT, build_model
from tests import refload


def _pair(n_layer=4, dupe=False, mtp=0.3, iha=True):
    ref = refload.load_limited(n_layer=n_layer, n_embd=128, n_head=4, seq_len=64, mtp_weight=mtp, iha=iha)
    if ref is None:
        pytest.skip("reference source not available")
    rcfg = ref.GPTConfig(sequence_len=64, vocab_size=50257, n_layer=n_layer, n_head=4, n_kv_head=4, n_embd=128,
                         dropout=0.0, stoch_depth=0.0, use_iha=iha, iha_mix_v=iha)
    torch.manual_seed(42)
    with torch.device("meta"):        # the script's own construction sequence (train.py:1044-1047)
        rmodel = ref.GPT(rcfg)
    rmodel.to_empty(device="cpu")
    rmodel.init_weights()
    mc = ModelConfig(sequence_len=64, n_layer=n_layer, n_head=4, n_kv_head=4, n_embd=128, dropout=0.0, stoch_depth=0.0,
                     use_iha=iha, iha_mix_v=iha, mtp_weight=mtp, logit_cap=10.0)
    model = build_model(mc, "cpu", seed=42)
    if dupe:
        rmodel.set_dupe_layers(n_layer // 2, n_layer // 2 + 1, 2)
        model.set_dupe_layers(n_layer // 2, n_layer // 2 + 1, 2)
    return ref, rmodel, model


def test_same_seed_gives_identical_parameters():
    _, rmodel, model = _pair()
    rp = dict(rmodel.named_parameters())
    mp = dict(model.named_parameters())
    assert list(rp.keys()) == list(mp.keys())
    for k in rp:
        assert rp[k].shape == mp[k].shape, k
        assert torch.equal(rp[k].detach(), mp[k].detach()), k


@pytest.mark.parametrize("dupe", [False, True])
def test_loss_and_grads_match_reference(dupe):
    _, rmodel, model = _pair(dupe=dupe)
    # perturb gates/mixes away from their zero/identity init so every path carries signal
    torch.manual_seed(1)
    with torch.no_grad():
        for (n, p), (_, q) in zip(rmodel.named_parameters(), model.named_parameters()):
            if "gate" in n or "mix" in n or "lambdas" in n or "skip" in n:
                d = torch.randn_like(p) * 0.05
                p.add_(d)
                q.add_(d)
    rmodel.train()
    model.train()
    idx = torch.randint(0, 50257, (2, 64))
    tgt = torch.randint(0, 50257, (2, 64))
    rl, rmet = rmodel(idx, tgt)
    ml, mmet = model(idx, tgt)
    assert torch.allclose(rl, ml, rtol=1e-5, atol=1e-5), (rl.item(), ml.item())
    assert torch.allclose(rmet["mtp_loss"], mmet["mtp_loss"], rtol=1e-5, atol=1e-5)
    rl.backward()
    ml.backward()
    for (n, p), (_, q) in zip(rmodel.named_parameters(), model.named_parameters()):
        g = model.arena.head_grad if n == "lm_head.weight" else q.grad
        assert torch.allclose(p.grad, g, rtol=2e-4, atol=2e-6), (n, (p.grad - g).abs().max().item())


def test_eval_paths_match_reference():
    _, rmodel, model = _pair()
    rmodel.eval()
    model.eval()
    idx = torch.randint(0, 50257, (2, 64))
    tgt = torch.randint(0, 50257, (2, 64))
    tgt[0, :5] = -1
    with torch.no_grad():
        assert torch.allclose(rmodel(idx), model(idx), rtol=1e-5, atol=1e-5)
        assert torch.allclose(rmodel(idx, tgt, loss_reduction="none"), model(idx, tgt, loss_reduction="none").view(-1), rtol=1e-5, atol=1e-5)


def test_flops_estimate_matches_reference():
    _, rmodel, model = _pair()
    assert rmodel.estimate_flops() == model.estimate_flops()


def test_checkpoint_roundtrip_into_reference_loader():
    ref, rmodel, model = _pair()
    from slowrun_b200.train.checkpoint import named_param_snapshot, load_named_params
    with torch.no_grad():
        for p in model.parameters():
            p.add_(0.01)
    snap = named_param_snapshot(model)
    # the reference's loader (train.py:182-186), verbatim semantics
    for name, p in rmodel.named_parameters():
        assert name in snap
        p.data.copy_(snap[name].to(p.device, dtype=p.dtype))
    idx = torch.randint(0, 50257, (1, 64))
    rmodel.eval(); model.eval()
    with torch.no_grad():
        assert torch.allclose(rmodel(idx), model(idx), rtol=1e-5, atol=1e-5)
    rsnap = {n: p.data.float().cpu() + 0.5 for n, p in rmodel.named_parameters()}
    load_named_params(model, rsnap)
    for n, p in model.named_parameters():
        assert torch.allclose(p.data.float(), rsnap[n])


# ------------------------------------------------------------------ tiny track (tiny/train.py:378-946)
def _tiny_pair(num_iterations=2):
    from slowrun_b200.config import track_defaults
    ref = refload.load_tiny(n_layer=4, n_embd=256, n_head=2, seq_len=64, num_iterations=num_iterations)
    if ref is None:
        pytest.skip("reference source not available")
    rcfg = ref.GPTConfig(sequence_len=64, vocab_size=50257, n_layer=4, n_head=2, n_kv_head=2, n_embd=256, dropout=0.0,
                         num_iterations=num_iterations)
    torch.manual_seed(42)
    with torch.device("meta"):
        rmodel = ref.GPT(rcfg)
    rmodel.to_empty(device="cpu")
    rmodel.init_weights()
    cfg = track_defaults("tiny")
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len, m.dropout, m.num_iterations = 4, 256, 2, 2, 64, 0.0, num_iterations
    model = build_model(m, "cpu", seed=42)
    # the tiny track starts with zero output projections, gates and XSA coefficients: move them (identically) so that every
    # path carries signal and no gradient is pure rounding noise
    torch.manual_seed(1)
    with torch.no_grad():
        for (n, p), (_, q) in zip(rmodel.named_parameters(), model.named_parameters()):
            if "c_proj" in n or "gate" in n or "xsa" in n or "lambdas" in n or "skip" in n:
                d = (torch.randn(p.shape) * (0.02 if "c_proj" in n else 0.05)).to(p.dtype)
                p.add_(d)
                q.add_(d)
    return ref, rmodel, model, cfg


def test_tiny_same_seed_gives_identical_parameters():
    ref = refload.load_tiny()
    if ref is None:
        pytest.skip("reference source not available")
    from slowrun_b200.config import track_defaults
    rcfg = ref.GPTConfig(sequence_len=64, vocab_size=50257, n_layer=4, n_head=2, n_kv_head=2, n_embd=256, dropout=0.0)
    torch.manual_seed(7)
    with torch.device("meta"):
        rmodel = ref.GPT(rcfg)
    rmodel.to_empty(device="cpu")
    rmodel.init_weights()
    cfg = track_defaults("tiny")
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 4, 256, 2, 2, 64
    model = build_model(m, "cpu", seed=7)
    rp, mp = dict(rmodel.named_parameters()), dict(model.named_parameters())
    assert list(rp) == list(mp)
    for k in rp:
        assert rp[k].dtype == mp[k].dtype and torch.equal(rp[k].detach(), mp[k].detach()), k


@pytest.mark.parametrize("iters", [1, 2])
def test_tiny_loss_and_grads_match_reference(iters):
    """Shifted-target multi-token loss through the shared head, XSA, key offset, truncated RoPE, recurrence with only the
    last pass back-propagated: loss and every gradient against the reference's tiny model."""
    _, rmodel, model, _ = _tiny_pair()
    rmodel.train()
    model.train()
    g = torch.Generator().manual_seed(0)
    idx = torch.randint(0, 50257, (2, 65), generator=g)
    x, y = idx[:, :-1], idx[:, 1:]
    w = torch.tensor([1.0, 0.5, 0.25])
    rl = rmodel(x, y, num_iterations=iters, mtp_weights=w).mean()
    ml = model(x, y, num_iterations=iters, mtp_weights=w)
    assert torch.allclose(rl, ml, rtol=1e-5, atol=1e-5), (rl.item(), ml.item())
    rl.backward()
    ml.backward()
    for (n, p), (_, q) in zip(rmodel.named_parameters(), model.named_parameters()):
        gq = q.grad if q.grad is not None else model.arena.head_grad
        rel = ((p.grad.float() - gq.float()).norm() / p.grad.float().norm().clamp_min(1e-20)).item()
        assert rel < 3e-3, (n, rel)


def test_tiny_first_optimizer_step_follows_reference():
    """One step of the reference's tiny optimizer against ours from identical gradients. Newton-Schulz maps every
    singular value to about one, so rounding-level differences in weak directions come back at the scale of the update;
    AdamW's first step is lr * sign(g), so only the sign pattern and the step size are comparable element by element."""
    ref, rmodel, model, cfg = _tiny_pair()
    from slowrun_b200.optim.groups import build_param_groups
    from slowrun_b200.optim.muon_adamw import ShardedMuonAdamW
    from slowrun_b200.parallel.comm import TorchComm
    ropt = rmodel.setup_optimizer()
    groups = build_param_groups(model, cfg)
    opt = ShardedMuonAdamW(model, groups, TorchComm())
    for grp in list(ropt.param_groups) + list(groups):
        if grp["kind"] == "muon":
            grp["momentum"] = 0.85
    rmodel.train()
    model.train()
    before = {n: p.detach().float().clone() for n, p in rmodel.named_parameters()}
    g = torch.Generator().manual_seed(0)
    idx = torch.randint(0, 50257, (2, 65), generator=g)
    w = torch.tensor([1.0, 0.5, 0.25])
    rmodel(idx[:, :-1], idx[:, 1:], num_iterations=1, mtp_weights=w).mean().backward()
    model(idx[:, :-1], idx[:, 1:], num_iterations=1, mtp_weights=w).backward()
    ropt.step()
    opt.step()
    for (n, p), (_, q) in zip(rmodel.named_parameters(), model.named_parameters()):
        pf, qf = p.detach().float(), q.detach().float()
        upd_r, upd_o = pf - before[n], qf - before[n]
        assert upd_r.norm() > 0, n
        if n in ("lm_head.weight", "transformer.wte.weight") or p.dim() < 2 or "attn_gate" in n:
            # AdamW: same step size, same direction for all but the elements whose gradient is rounding noise
            assert abs(upd_o.norm().item() / upd_r.norm().item() - 1) < 0.05, n
            moved = upd_r != 0
            agree = (upd_r.sign() == upd_o.sign())[moved].float().mean().item()
            assert agree > 0.95, (n, agree)
        else:
            assert ((pf - qf).norm() / pf.norm()).item() < 2e-2, n
            cos = (upd_r.flatten() @ upd_o.flatten() / (upd_r.norm() * upd_o.norm())).item()
            assert cos > 0.97, (n, cos)
