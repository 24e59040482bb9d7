"""One optimizer step of ShardedMuonAdamW (single process, CPU) against the reference's muon_step_fused /
adamw_step_fused run eagerly (train.py:594-639), plus the grouping rules."""
import pytest
import torch

from slowrun_b200.config import track_defaults
from slowrun_b200.models.gpt import build_model
from slowrun_b200.optim.groups import build_param_groups
from slowrun_b200.optim.muon_adamw import ShardedMuonAdamW, muon_update_ref, muon_apply_ref, POLAR_EXPRESS_COEFFS
from slowrun_b200.parallel.comm import TorchComm
from tests import refload


def _small_cfg(track="limited"):
    cfg = track_defaults(track)
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 4, 128, 4, 4, 64
    m.dropout, m.stoch_depth = 0.0, 0.0
    return cfg


def test_groups_match_reference_membership_and_order():
    ref = refload.load_limited()
    if ref is None:
        pytest.skip("reference source not available")
    cfg = _small_cfg()
    model = build_model(cfg.model, "cpu")
    groups = build_param_groups(model, cfg)
    rcfg = ref.GPTConfig(sequence_len=64, vocab_size=50257, n_layer=4, n_head=4, n_kv_head=4, n_embd=128,
                         dropout=0.0, stoch_depth=0.0, use_iha=True, iha_mix_v=True)
    rmodel = ref.GPT(rcfg)

    class _Opt:
        def __init__(self, pg):
            self.param_groups = pg
    ref.DistMuonAdamW = _Opt
    rmodel.setup_optimizer.__globals__["DistMuonAdamW"] = _Opt
    ropt = rmodel.setup_optimizer()
    rname = {id(p): n for n, p in rmodel.named_parameters()}
    mname = {id(p): n for n, p in model.named_parameters()}
    rgroups = [g for g in ropt.param_groups if len(g["params"]) > 0]
    assert len(rgroups) == len(groups)
    for rg, g in zip(rgroups, groups):
        assert rg["kind"] == g["kind"]
        assert [rname[id(p)] for p in rg["params"]] == [mname[id(p)] for p in g["params"]]
        # reference LRs were built with lr_multiplier folded in by the caller; compare the ratios that matter
        assert rg["weight_decay"] == pytest.approx(g["weight_decay"])


@pytest.mark.parametrize("shape", [(3, 64, 32), (2, 32, 96), (2, 48, 48)])
def test_muon_math_matches_reference(shape):
    ref = refload.load_limited()
    if ref is None:
        pytest.skip("reference source not available")
    torch.manual_seed(0)
    n, r, c = shape
    G = torch.randn(n, r, c) * 0.02
    P = torch.randn(n, r, c) * 0.05
    M = torch.randn(n, r, c) * 0.01
    S = torch.rand(n, r, 1) * 1e-3 if r >= c else torch.rand(n, 1, c) * 1e-3
    lr, wd, mu, b2 = 0.02, 1.3, 0.9, 0.95
    # reference, eager
    rG, rP, rM, rS = G.clone(), P.clone(), M.clone(), S.clone()
    red_dim = -1 if r >= c else -2
    ref.muon_step_fused(rG, rP, rM, rS, torch.tensor(mu), torch.tensor(lr), torch.tensor(wd), torch.tensor(b2), 5, red_dim)
    # ours
    mG, mP, mM, mS = G.clone(), P.clone(), M.clone(), S.clone()
    U = muon_update_ref(mG, mM, mS, mu, b2, 5)
    muon_apply_ref(mP, U, lr, wd)
    assert torch.allclose(rM, mM, rtol=1e-6, atol=1e-8)
    assert torch.allclose(rS, mS, rtol=2e-2, atol=1e-7)
    # bf16 Newton-Schulz amplifies last-bit differences; the applied update must agree to bf16 accuracy
    assert torch.allclose(rP, mP, rtol=0, atol=lr * 0.05), (rP - mP).abs().max().item()
    rel = (rP - mP).norm() / (rP - P).norm()
    assert rel < 0.03, rel.item()


def test_adamw_matches_reference():
    ref = refload.load_limited()
    if ref is None:
        pytest.skip("reference source not available")
    from slowrun_b200.optim.muon_adamw import adamw_ref
    torch.manual_seed(0)
    p = torch.randn(64, 32); g = torch.randn(64, 32) * 0.1
    m = torch.randn(64, 32) * 0.01; v = torch.rand(64, 32) * 0.01
    rp, rm, rv = p.clone(), m.clone(), v.clone()
    t = lambda x: torch.tensor(float(x))
    ref.adamw_step_fused(rp, g, rm, rv, t(3), t(0.01), t(0.8), t(0.95), t(1e-10), t(1.3))
    adamw_ref(p, g, m, v, 3, 0.01, 0.8, 0.95, 1e-10, 1.3)
    assert torch.allclose(rp, p, rtol=1e-6, atol=1e-7)
    assert torch.allclose(rm, m) and torch.allclose(rv, v)


def test_full_step_runs_and_changes_every_parameter():
    cfg = _small_cfg()
    torch.manual_seed(0)
    model = build_model(cfg.model, "cpu")
    groups = build_param_groups(model, cfg)
    opt = ShardedMuonAdamW(model, groups, TorchComm())
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    idx = torch.randint(0, 50257, (2, 64)); tgt = torch.randint(0, 50257, (2, 64))
    # two steps: zero-initialised gates block some gradients on the very first one
    for _ in range(2):
        loss, _ = model(idx, tgt)
        loss.backward()
        opt.step()
        model.zero_grad_arena()
    unchanged = [n for n, p in model.named_parameters() if torch.equal(before[n], p.detach())]
    assert unchanged == [], unchanged
    for p in model.parameters():
        assert torch.isfinite(p).all()


def test_tiny_groups():
    cfg = _small_cfg("tiny")
    model = build_model(cfg.model, "cpu")
    groups = build_param_groups(model, cfg)
    names = [g["name"] for g in groups if g["kind"] == "adamw"]
    assert names == ["lm_head", "wte", "resid", "x0", "skip", "attn_gate", "xsa"]
    muon_shapes = [tuple(g["params"][0].shape) for g in groups if g["kind"] == "muon"]
    assert (4, 12) not in muon_shapes and (4, 32) in muon_shapes


@pytest.mark.parametrize("shape", [(3, 64, 32), (2, 32, 96)])
def test_tiny_muon_math_matches_reference_including_the_active_mask(shape):
    """tiny/train.py:770-809: no row normalisation before Newton-Schulz, and a matrix whose mask is off keeps its
    parameter, momentum and second moment."""
    ref = refload.load_tiny_optimizer()
    if ref is None:
        pytest.skip("reference source not available")
    torch.manual_seed(0)
    n, r, c = shape
    G = torch.randn(n, r, c) * 0.02
    P = torch.randn(n, r, c) * 0.05
    M = torch.randn(n, r, c) * 0.01
    S = torch.rand(n, r, 1) * 1e-3 if r >= c else torch.rand(n, 1, c) * 1e-3
    lr, wd, mu, b2 = 0.02, 0.8, 0.9, 0.95
    active = torch.ones(n, 1, 1, dtype=torch.bool)
    active[1] = False
    rG, rP, rM, rS = G.clone(), P.clone(), M.clone(), S.clone()
    rG[1].zero_()
    red_dim = -1 if r >= c else -2
    ref.muon_step_fused(rG, rP, rM, rS, torch.tensor(mu), torch.tensor(lr), torch.tensor(wd), torch.tensor(b2), active, 5, red_dim)
    # ours: the inactive matrix is left out of the call
    mP, mM, mS = P.clone(), M.clone(), S.clone()
    for i in (0,) + tuple(range(2, n)):
        U = muon_update_ref(G[i:i + 1].clone(), mM[i:i + 1], mS[i:i + 1], mu, b2, 5, row_norm=False)
        muon_apply_ref(mP[i:i + 1], U, lr, wd)
    assert torch.equal(rP[1], P[1]) and torch.equal(rM[1], M[1]) and torch.equal(rS[1], S[1])
    assert torch.equal(mP[1], P[1])
    assert torch.allclose(rM, mM, rtol=1e-6, atol=1e-8)
    assert torch.allclose(rS, mS, rtol=2e-2, atol=1e-7)
    rel = (rP - mP).norm() / (rP - P).norm()
    assert rel < 0.03, rel.item()
    # and the row-normalised variant is measurably different, so the switch is not a no-op
    U_rn = muon_update_ref(G[:1].clone(), M[:1].clone(), S[:1].clone(), mu, b2, 5, row_norm=True)
    U_no = muon_update_ref(G[:1].clone(), M[:1].clone(), S[:1].clone(), mu, b2, 5, row_norm=False)
    assert (U_rn.float() - U_no.float()).norm() / U_no.float().norm() > 0.02


def test_tiny_track_groups_skip_row_norm_and_inactive_parameters_are_left_alone():
    cfg = _small_cfg("tiny")
    torch.manual_seed(0)
    model = build_model(cfg.model, "cpu")
    groups = build_param_groups(model, cfg)
    assert all(g["row_norm"] is False for g in groups if g["kind"] == "muon")
    assert all(g["row_norm"] is True for g in build_param_groups(build_model(_small_cfg().model, "cpu"), _small_cfg()) if g["kind"] == "muon")
    opt = ShardedMuonAdamW(model, groups, TorchComm())
    frozen = [model.transformer.h[1].mlp.c_fc.weight, model.transformer.h[2].attn.c_q.weight, model.x0_lambdas]
    opt.set_inactive(frozen)
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    idx = torch.randint(0, 50257, (2, 64)); tgt = torch.randint(0, 50257, (2, 64))
    for _ in range(2):
        loss = model(idx, tgt, num_iterations=1, mtp_weights=torch.tensor([1.0, 0.5, 0.25]))
        loss.backward()
        opt.step()
        model.zero_grad_arena()
    frozen_ids = {id(p) for p in frozen}
    for n, p in model.named_parameters():
        same = torch.equal(before[n], p.detach())
        assert same == (id(p) in frozen_ids), n
