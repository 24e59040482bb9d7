"""The research forks end to end on CPU: gated delta rule (chunked form vs the token-by-token definition, values and
gradients), the hybrid and universal-transformer trainers through their entry scripts on a tiny synthetic corpus."""
import importlib.util
import json
import os

import pytest
import torch

from slowrun_b200.data.synthetic import write_synthetic_corpus
from slowrun_b200.ops.linear_attention import gated_delta_rule_chunked, gated_delta_rule_recurrent

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def corpus(tmp_path_factory):
    d = tmp_path_factory.mktemp("corpus")
    return write_synthetic_corpus(str(d), train_tokens=70_000, val_tokens=20_000)


@pytest.mark.parametrize("per_channel", [False, True])
@pytest.mark.parametrize("T,chunk", [(37, 16), (64, 64), (50, 8)])
def test_chunked_gated_delta_rule_equals_the_recurrence(per_channel, T, chunk):
    torch.manual_seed(0)
    B, H, Dk, Dv = 2, 3, 8, 5
    q, k, v = torch.randn(B, T, H, Dk), torch.nn.functional.normalize(torch.randn(B, T, H, Dk), dim=-1), torch.randn(B, T, H, Dv)
    g = -torch.rand(B, T, H, Dk) * 3 if per_channel else -torch.rand(B, T, H) * 3      # strong decays included
    beta = torch.rand(B, T, H) * 2
    ins = [t.double().requires_grad_(True) for t in (q, k, v, g, beta)]
    o_ref = gated_delta_rule_recurrent(*ins)
    w = torch.randn_like(o_ref)
    g_ref = torch.autograd.grad((o_ref.float() * w).sum(), ins)
    ins2 = [t.detach().clone().requires_grad_(True) for t in ins]
    o = gated_delta_rule_chunked(*ins2, chunk_size=chunk)
    g_new = torch.autograd.grad((o.float() * w).sum(), ins2)
    assert torch.allclose(o.float(), o_ref.float(), atol=2e-4, rtol=1e-3)
    for a, b in zip(g_new, g_ref):
        assert torch.allclose(a.float(), b.float(), atol=5e-4, rtol=2e-3), (a - b).abs().max()


def test_chunk_states_chain():
    """Running two halves with the state handed over equals one run over the whole sequence."""
    torch.manual_seed(1)
    B, T, H, Dk, Dv = 1, 40, 2, 8, 8
    q, k, v = torch.randn(B, T, H, Dk), torch.nn.functional.normalize(torch.randn(B, T, H, Dk), dim=-1), torch.randn(B, T, H, Dv)
    g, beta = -torch.rand(B, T, H), torch.rand(B, T, H)
    full = gated_delta_rule_chunked(q, k, v, g, beta, chunk_size=16)
    a, S = gated_delta_rule_chunked(q[:, :24], k[:, :24], v[:, :24], g[:, :24], beta[:, :24], chunk_size=16, return_state=True)
    b = gated_delta_rule_chunked(q[:, 24:], k[:, 24:], v[:, 24:], g[:, 24:], beta[:, 24:], chunk_size=16, initial_state=S)
    assert torch.allclose(torch.cat([a, b], 1), full, atol=1e-5)


@pytest.mark.parametrize("kind", ["gdn", "kda"])
def test_linear_attention_layers_are_causal_and_trainable(kind):
    from slowrun_b200.config import ModelConfig
    from slowrun_b200.models.hybrid import GatedDeltaNetAttention, HybridSpec, KimiDeltaAttention
    torch.manual_seed(0)
    mc = ModelConfig(n_layer=2, n_head=2, n_kv_head=2, n_embd=256, sequence_len=32, dropout=0.0)
    cls = GatedDeltaNetAttention if kind == "gdn" else KimiDeltaAttention
    layer = cls(mc, HybridSpec(layers=[0], kind=kind), 0)
    layer.reset_parameters(3 ** 0.5 * 256 ** -0.5)
    torch.nn.init.normal_(layer.o_proj.weight, std=0.05)
    x = torch.randn(1, 12, 256)
    y1 = layer(x)
    x2 = x.clone()
    x2[:, 7:] += 1.0
    assert torch.allclose(layer(x2)[:, :7], y1[:, :7], atol=1e-5)        # later tokens cannot influence earlier outputs
    y1.square().mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in layer.parameters())
    names = {n for n, _ in layer.named_parameters()}
    want = {"qk_proj.weight", "vg_proj.weight", "beta_bias"} if kind == "gdn" else {"f_proj.0.weight", "g_proj.1.weight", "dt_bias"}
    assert want <= names


def test_hybrid_entry_script_trains_clips_averages_and_blends(corpus, tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    mod = _load("research/hybrid_attn/train.py", "hybrid_train")
    out = tmp_path / "res.json"
    res = mod.main(["--n_layer", "4", "--n_head", "2", "--n_embd", "256", "--sequence-len", "64", "--device-batch-size", "2",
                    "--total-batch-size", "256", "--num-epochs", "2", "--gdn-layers", "1,2", "--grad-clip", "1.0",
                    "--ema-start-frac", "0.3", "--checkpoint-avg", "2", "--dupe-start-epoch", "2", "--dupe-layers-start", "2",
                    "--dupe-layers-end", "3", "--dropout", "0.0", "--input_bin", corpus[0], "--input_val_bin", corpus[1],
                    "--eval-tokens", "512", "--max-steps", "60", "--muon-ns-schedule", "deepseek-v4", "--no-muon-eq-r",
                    "--gdn-profile", "--save-result", str(out), "--run", "hybrid_cpu"])
    assert res["steps"] > 10 and res["final_train_loss"] < 11.0
    saved = json.loads(out.read_text())
    assert saved["best_val_loss"] <= saved["val_loss"] + 1e-9


def test_hybrid_kda_model_steps_on_the_sharded_optimizer(corpus, tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    mod = _load("research/hybrid_attn/train.py", "hybrid_train_kda")
    res = mod.main(["--n_layer", "2", "--n_head", "2", "--n_embd", "256", "--sequence-len", "64", "--device-batch-size", "2",
                    "--total-batch-size", "256", "--num-epochs", "1", "--gdn-layers", "0", "--linear-attn-type", "kda",
                    "--ema-decays", "", "--dropout", "0.0", "--input_bin", corpus[0], "--input_val_bin", corpus[1],
                    "--eval-tokens", "512", "--max-steps", "6", "--run", "kda_cpu"])
    assert res["steps"] == 6


def test_universal_entry_script_grows_depth_and_keeps_idle_layers_untouched(corpus, tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    mod = _load("research/universal_transformer/train.py", "ut_train")
    args = mod.build_parser().parse_args([
        "--n_head", "2", "--n_embd", "64", "--sequence-len", "64", "--device-batch-size", "2", "--total-batch-size", "256",
        "--num-epochs", "1", "--n-layer-schedule", "0:2,5:4", "--dropout", "0.0", "--stoch-depth", "0.0", "--logit-avg", "0",
        "--input_bin", corpus[0], "--input_val_bin", corpus[1], "--eval-tokens", "512", "--max-steps", "8", "--run", "ut_cpu"])
    cfg, uc = mod.configs_from(args)
    from slowrun_b200.train.research import UniversalTrainer
    tr = UniversalTrainer(cfg, uc, quiet=True)
    model = tr.model
    assert model.active_n_layer == 2
    idle = {n: p.detach().clone() for n, p in model.named_parameters() if any(p is q for q in model.inactive_parameters())}
    assert idle, "with 2 of 4 layers active some per-layer parameters must be idle"
    for _ in range(4):
        tr.train_step()
    assert all(torch.equal(dict(model.named_parameters())[n].detach(), v) for n, v in idle.items())
    for _ in range(3):
        tr.train_step()
    assert model.active_n_layer == 4 and not model.inactive_parameters()
    tr.train_step()
    changed = [n for n, v in idle.items() if not torch.equal(dict(model.named_parameters())[n].detach(), v)]
    assert changed, "after the depth grew the formerly idle layers are trained"
