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
