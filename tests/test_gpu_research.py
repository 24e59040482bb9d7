"""The research forks on a GPU: a few optimizer steps of the hybrid model (Gated DeltaNet and Kimi Delta Attention layers on
the CUDA recurrence kernel, softmax layers on the fused block node) and of the universal transformer through their entry
scripts, and the hybrid model's first loss and gradients against the same model on the CPU."""
import importlib.util
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def corpus(tmp_path_factory):
    from slowrun_b200.data.synthetic import write_synthetic_corpus
    return write_synthetic_corpus(str(tmp_path_factory.mktemp("corpus")), train_tokens=60_000, val_tokens=8_000)


@pytest.mark.parametrize("kind", ["gdn", "kda"])
def test_hybrid_entry_script_trains_on_gpu(kind, corpus, tmp_path, monkeypatch):
    from slowrun_b200.ops import _lib
    monkeypatch.chdir(tmp_path)
    mod = _load("research/hybrid_attn/train.py", f"hybrid_gpu_{kind}")
    res = mod.main(["--n_layer", "4", "--n_head", "2", "--n_embd", "256", "--sequence-len", "256", "--device-batch-size", "2",
                    "--total-batch-size", "1024", "--num-epochs", "1", "--gdn-layers", "1,2", "--linear-attn-type", kind,
                    "--grad-clip", "1.0", "--ema-decays", "", "--dropout", "0.0", "--input_bin", corpus[0], "--input_val_bin",
                    corpus[1], "--eval-tokens", "2048", "--max-steps", "12", "--run", f"hybrid_gpu_{kind}"])
    torch.cuda.synchronize()
    _lib.check_status()
    assert res["steps"] == 12 and res["final_train_loss"] < 10.9, res


def test_universal_entry_script_trains_on_gpu(corpus, tmp_path, monkeypatch):
    from slowrun_b200.ops import _lib
    monkeypatch.chdir(tmp_path)
    mod = _load("research/universal_transformer/train.py", "ut_gpu")
    args = mod.build_parser().parse_args([
        "--n_head", "2", "--n_embd", "256", "--sequence-len", "256", "--device-batch-size", "2", "--total-batch-size", "1024",
        "--num-epochs", "1", "--n-layer-schedule", "0:2,5:4", "--dropout", "0.0", "--stoch-depth", "0.0", "--logit-avg", "0",
        "--input_bin", corpus[0], "--input_val_bin", corpus[1], "--eval-tokens", "2048", "--max-steps", "10", "--run", "ut_gpu"])
    cfg, uc = mod.configs_from(args)
    from slowrun_b200.train.research import UniversalTrainer
    tr = UniversalTrainer(cfg, uc, quiet=True)
    first = tr.train_step()["loss"]
    for _ in range(9):
        last = tr.train_step()["loss"]
    torch.cuda.synchronize()
    _lib.check_status()
    assert tr.model.active_n_layer == 4 and last < first


def test_hybrid_model_matches_its_cpu_path():
    """Same weights on both devices: the GPU forward (CUDA recurrence, fused softmax blocks, bf16 GEMMs) against the fp32 CPU
    path, and the gradients of the linear-attention parameters."""
    from slowrun_b200.config import track_defaults
    from slowrun_b200.models.gpt import build_model
    from slowrun_b200.models.hybrid import HybridGPT, HybridSpec
    cfg = track_defaults("limited")
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len, m.dropout, m.stoch_depth = 4, 256, 2, 2, 128, 0.0, 0.0
    spec = HybridSpec(layers=[1, 2], kind="gdn")
    make = lambda c: HybridGPT(c, spec)       # noqa: E731
    cpu = build_model(m, "cpu", seed=3, factory=make)
    gpu = build_model(m, "cuda", seed=3, factory=make)
    with torch.no_grad():
        for (n, p), (_, q) in zip(cpu.named_parameters(), gpu.named_parameters()):
            q.copy_(p.to(q.dtype))
            if "o_proj" in n or "c_proj" in n:                      # zero-initialised in the fork: give them signal
                d = torch.randn(p.shape, generator=torch.Generator().manual_seed(len(n))) * 0.02
                p.add_(d)
                q.add_(d.to(q.device, q.dtype))
    gpu.arena.refresh_shadows()
    idx = torch.randint(0, 50257, (2, 129), generator=torch.Generator().manual_seed(0))
    lc, _ = cpu(idx[:, :-1], idx[:, 1:])
    lg, _ = gpu(idx[:, :-1].cuda(), idx[:, 1:].cuda())
    assert abs(lc.item() - lg.item()) < 3e-2, (lc.item(), lg.item())
    lc.backward()
    lg.backward()
    for (n, p), (_, q) in zip(cpu.named_parameters(), gpu.named_parameters()):
        if "transformer.h.1.attn" in n and p.grad is not None and q.grad is not None and p.grad.norm() > 1e-6:
            cos = torch.nn.functional.cosine_similarity(p.grad.flatten().float(), q.grad.flatten().float().cpu(), dim=0).item()
            assert cos > 0.98, (n, cos)
