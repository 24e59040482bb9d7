"""Whole-run GPU checks of the track drivers through `Trainer.fit()` on a small model: the two-hour track across a window
stage (longer long window, YaRN rescaling, CUDA graphs captured again for the new kernel arguments), the tiny track with
recurrence switch, weight EMA and checkpoint averaging, and the limited track with layer replay and probability averaging."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(track, tmp_path, corpus):
    from slowrun_b200.config import track_defaults
    cfg = track_defaults(track)
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 4, 256, 2, 2, 256
    cfg.device_batch_size, cfg.total_batch_size, cfg.eval_tokens = 4, 4 * 256 * 2, 4 * 256 * 2
    cfg.input_bin, cfg.input_val_bin = corpus
    cfg.runs_dir, cfg.logit_avg_dir, cfg.run_name = str(tmp_path / "runs"), str(tmp_path / "ring"), "t"
    return cfg


@pytest.fixture(scope="module")
def corpus(tmp_path_factory):
    from slowrun_b200.data.synthetic import write_synthetic_corpus
    return write_synthetic_corpus(str(tmp_path_factory.mktemp("corpus")), train_tokens=50_000, val_tokens=12_000)


def _info():
    from slowrun_b200.parallel.comm import DistInfo
    return DistInfo(False, 0, 0, 1, torch.device("cuda", 0))


def _done():
    from slowrun_b200.ops import _lib
    torch.cuda.synchronize()
    _lib.check_status()


def test_two_hour_track_crosses_a_window_stage(corpus, tmp_path):
    from slowrun_b200.train.trainer import Trainer
    cfg = _cfg("two_hour", tmp_path, corpus)
    cfg.num_epochs, cfg.swa_last_epochs, cfg.logit_avg, cfg.dupe_start_epoch = 2, 1, 2, 2
    cfg.dupe_layers_start, cfg.dupe_layers_end = 2, 3
    cfg.window_schedule = "1-1:64,128;2-2:128,256"
    tr = Trainer(cfg, _info(), quiet=True)
    s0 = tr.model.rotary.attn_scale
    res = tr.fit()
    _done()
    assert tr.model.long_window == 256 and tr.model.rotary.yarn_active and tr.model.rotary.attn_scale > s0
    assert tr.dupe_active and res["steps"] > 20 and res["best_val_loss"] < 10.9
    assert len(tr._graphs) >= 2, "the window stage and the layer replay each need their own captured micro-step"


def test_tiny_track_runs_recurrence_ema_and_checkpoint_average(corpus, tmp_path):
    from slowrun_b200.train.trainer import Trainer
    cfg = _cfg("tiny", tmp_path, corpus)
    cfg.device_batch_size, cfg.total_batch_size, cfg.eval_tokens = 4, 4 * 256, 4 * 256 * 2
    cfg.num_epochs, cfg.swa_last_epochs, cfg.update_ema_every, cfg.max_train_steps = 3, 2, 2, 0
    cfg.iteration_transition_ratio = 0.5
    tr = Trainer(cfg, _info(), quiet=True)
    res = tr.fit()
    _done()
    assert res["steps"] > 30 and res["best_val_loss"] < 10.9
    assert tr.sched.num_recurrences(res["steps"] - 1) == 2 and tr.sched.num_recurrences(0) == 1
    assert os.path.exists(os.path.join(cfg.runs_dir, "t", "model.pt"))


def test_limited_track_probability_averaging(corpus, tmp_path):
    from slowrun_b200.train.trainer import Trainer
    cfg = _cfg("limited", tmp_path, corpus)
    cfg.num_epochs, cfg.swa_last_epochs, cfg.logit_avg, cfg.dupe_start_epoch = 3, 2, 2, 2
    cfg.dupe_layers_start, cfg.dupe_layers_end = 2, 3
    tr = Trainer(cfg, _info(), quiet=True)
    res = tr.fit()
    _done()
    assert tr.dupe_active and len(os.listdir(cfg.logit_avg_dir)) == 2 and res["best_val_loss"] < 10.9
