"""The unlimited track on a GPU: a chain of three snapshots (perturbation, distillation from the previous snapshot through the
soft-capped logits kernel path, target-probability cache, greedy selection, single-pass ensemble evaluation) and a resume
from its cycle file."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_unlimited_chain_runs_distills_selects_and_resumes_on_gpu(tmp_path):
    from slowrun_b200.config import track_defaults
    from slowrun_b200.data.synthetic import write_synthetic_corpus
    from slowrun_b200.ops import _lib
    from slowrun_b200.parallel.comm import DistInfo
    from slowrun_b200.train.unlimited import UnlimitedTrainer
    corpus = write_synthetic_corpus(str(tmp_path / "data"), train_tokens=120_000, val_tokens=16_000)
    cfg = track_defaults("unlimited")
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 4, 256, 2, 2, 256
    cfg.device_batch_size, cfg.total_batch_size, cfg.bs_floor = 4, 4 * 256 * 2, 4 * 256 * 2
    cfg.eval_tokens = 4 * 256 * 2
    cfg.input_bin, cfg.input_val_bin = corpus
    cfg.runs_dir = str(tmp_path / "runs")
    cfg.num_models, cfg.epochs_per_cycle, cfg.distill_after_cycles = 3, 0.1, 1
    cfg.fitness_tokens, cfg.pgt_steps, cfg.k_sweep, cfg.grad_opt_steps = 4096, 2, (2, 3), 30
    cfg.checkpoint_base, cfg.run_name = str(tmp_path / "ck"), "u"
    cfg.dupe_layers_start, cfg.dupe_layers_end, cfg.dupe_loops = 2, 3, 1
    info = DistInfo(False, 0, 0, 1, torch.device("cuda", 0))
    tr = UnlimitedTrainer(cfg, info)
    out = tr.run()
    torch.cuda.synchronize()
    _lib.check_status()
    assert len(out["models"]) == 3 and set(out["ensemble"]) == {2, 3}
    assert all(os.path.exists(os.path.join(cfg.checkpoint_base, "u", f"model_{i}.pt")) for i in range(3))
    losses = [r["val_loss"] for r in out["models"]]
    assert losses[2] < losses[0], losses                       # the chain learns (each snapshot starts from the previous one)
    # the ensemble of all three lies between the best and the worst member (six-step models of very different quality)
    assert min(losses) - 0.5 < out["ensemble"][3]["val_loss"] < max(losses)
    assert abs(sum(out["selection"][2]["weights"]) - 1.0) < 1e-5
    cfg.resume = "u"
    tr2 = UnlimitedTrainer(cfg, info)
    assert tr2.try_resume() and tr2.cycle == 3 and len(tr2.results) == 3
