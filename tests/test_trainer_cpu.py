"""End-to-end CPU runs of the training drivers on a tiny model and a tiny synthetic corpus: the loop, schedules,
epoch handling, checkpoint ring, averaging passes, tiny-track recurrence/MTP/EMA and the unlimited chain."""
import json
import os

import pytest
import torch

from slowrun_b200.config import track_defaults, config_from_args
from slowrun_b200.data.synthetic import write_synthetic_corpus
from slowrun_b200.parallel.comm import DistInfo


@pytest.fixture(scope="module")
def corpus(tmp_path_factory):
    d = tmp_path_factory.mktemp("corpus")
    return write_synthetic_corpus(str(d), train_tokens=24_000, val_tokens=8_000)


def _shrink(cfg, corpus, tmp_path):
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 2, 64, 2, 2, 64
    cfg.device_batch_size = 4
    cfg.total_batch_size = 4 * 64 * 2
    cfg.eval_tokens = 4 * 64 * 2
    cfg.input_bin, cfg.input_val_bin = corpus
    cfg.runs_dir = str(tmp_path / "runs")
    cfg.logit_avg_dir = str(tmp_path / "ckpts")
    cfg.run_name = "t"
    return cfg


def _info():
    return DistInfo(False, 0, 0, 1, torch.device("cpu"))


def test_limited_track_runs_epochs_checkpoints_and_logit_average(corpus, tmp_path):
    from slowrun_b200.train.trainer import Trainer
    cfg = _shrink(track_defaults("limited"), corpus, tmp_path)
    cfg.num_epochs, cfg.swa_last_epochs, cfg.logit_avg, cfg.dupe_start_epoch = 3, 2, 2, 2
    cfg.dupe_layers_start, cfg.dupe_layers_end = 1, 2
    tr = Trainer(cfg, _info(), quiet=True)
    res = tr.fit()
    assert tr.dupe_active and tr.current_epoch > 3
    assert res["steps"] > 0 and res["best_val_loss"] < 11.0
    assert len(os.listdir(cfg.logit_avg_dir)) == 2
    ck = torch.load(os.path.join(cfg.logit_avg_dir, sorted(os.listdir(cfg.logit_avg_dir))[-1]), weights_only=True)
    assert set(ck) == {n for n, _ in tr.model.named_parameters()} and all(v.dtype == torch.float32 for v in ck.values())
    assert json.load(open(os.path.join(cfg.runs_dir, "t", "result.json")))["steps"] == res["steps"]


def test_two_hour_window_schedule_applies_yarn(corpus, tmp_path):
    from slowrun_b200.train.trainer import Trainer
    cfg = _shrink(track_defaults("two_hour"), corpus, tmp_path)
    cfg.num_epochs, cfg.swa_last_epochs, cfg.logit_avg, cfg.dupe_start_epoch = 2, 0, 0, 99
    cfg.window_schedule = "1-1:16,32;2-2:32,64"
    tr = Trainer(cfg, _info(), quiet=True)
    assert tr.model.long_window == 32
    s0 = tr.model.rotary.attn_scale
    tr.fit()
    assert tr.model.long_window == 64 and tr.model.rotary.yarn_active and tr.model.rotary.attn_scale > s0


def test_tiny_track_recurrence_mtp_ema_and_weight_average(corpus, tmp_path):
    from slowrun_b200.train.trainer import Trainer
    cfg = _shrink(track_defaults("tiny"), corpus, tmp_path)
    cfg.num_epochs, cfg.swa_last_epochs, cfg.update_ema_every, cfg.max_train_steps = 3, 2, 2, 0
    tr = Trainer(cfg, _info(), quiet=True)
    assert tr.sched.num_recurrences(0) == 1 and tr.sched.num_recurrences(tr.sched.N) == 2
    assert tr.sched.mtp_weights(0) == [1.0, 0.5, 0.25] and tr.sched.mtp_weights(tr.sched.N)[1:] == [0.0, 0.0]
    res = tr.fit()
    assert tr.ema.updates > 0 and res["best_val_loss"] < 11.0
    assert os.path.exists(os.path.join(cfg.runs_dir, "t", "model.pt"))


def test_reference_flag_spellings_are_accepted():
    cfg = config_from_args("limited", ["--n_embd", "2560", "--n_head", "20", "--device-batch-size", "2", "--no-iha",
                                       "--output_json", "x.json", "--dupe-loops", "3", "--logit-avg-mode", "equal"])
    assert cfg.model.n_embd == 2560 and cfg.model.n_head == 20 and not cfg.model.use_iha and cfg.save_result == "x.json"
    t = config_from_args("tiny", ["--xsa-mode", "first6", "--wd-mid", "0.2", "--mtp-predict", "2"])
    assert t.model.xsa_mode == "first6" and t.wd_mid == 0.2 and t.mtp_predict == 2
    u = config_from_args("unlimited", ["--num-models", "4", "--k-sweep", "2", "4", "--run", "r1", "--distill-alpha", "0.3"])
    assert u.num_models == 4 and list(u.k_sweep) == [2, 4] and u.run_name == "r1" and u.distill_alpha == 0.3
    h = config_from_args("two_hour", [])
    assert h.num_epochs == 22 and h.window_schedule.startswith("1-6:256,768")


def test_unlimited_chain_distills_selects_and_resumes(corpus, tmp_path):
    from slowrun_b200.train.unlimited import UnlimitedTrainer
    cfg = _shrink(track_defaults("unlimited"), corpus, tmp_path)
    cfg.num_models, cfg.epochs_per_cycle, cfg.distill_after_cycles = 3, 0.1, 1
    cfg.bs_floor = cfg.total_batch_size
    cfg.fitness_tokens, cfg.pgt_steps, cfg.k_sweep, cfg.grad_opt_steps = 2000, 2, (2, 3), 30
    cfg.checkpoint_base, cfg.run_name = str(tmp_path / "ck"), "u"
    cfg.dupe_layers_start, cfg.dupe_layers_end, cfg.dupe_loops = 1, 2, 1
    tr = UnlimitedTrainer(cfg, _info())
    out = tr.run()
    assert len(out["models"]) == 3 and set(out["ensemble"]) == {2, 3}
    assert all(os.path.exists(os.path.join(cfg.checkpoint_base, "u", f"model_{i}.pt")) for i in range(3))
    assert out["ensemble"][3]["val_loss"] < 11.0
    assert abs(sum(out["selection"][2]["weights"]) - 1.0) < 1e-5
    # resume: a fresh trainer picks up after the last finished cycle and goes straight to selection
    cfg.resume = "u"
    tr2 = UnlimitedTrainer(cfg, _info())
    assert tr2.try_resume() and tr2.cycle == 3 and len(tr2.results) == 3


def test_resume_continues_bit_for_bit(corpus, tmp_path):
    """Six steps in one go against three steps, a resume file, a fresh process-like trainer and three more: same
    parameters, same optimizer state, same batches (dropout on, so the RNG streams are part of the state)."""
    from slowrun_b200.train.trainer import Trainer

    def make(sub):
        cfg = _shrink(track_defaults("limited"), corpus, tmp_path / sub)
        cfg.num_epochs, cfg.swa_last_epochs, cfg.logit_avg, cfg.dupe_start_epoch = 4, 0, 0, 2
        cfg.dupe_layers_start, cfg.dupe_layers_end = 1, 2
        cfg.model.dropout = 0.1
        torch.manual_seed(1234)
        return Trainer(cfg, _info(), quiet=True)

    a = make("a")
    losses_a = [a.train_step()["loss"] for _ in range(6)]
    b = make("b")
    losses_b = [b.train_step()["loss"] for _ in range(3)]
    b.current_epoch = b._pending_epoch
    path = str(tmp_path / "resume" / "state")
    b.save_state(path, {"min_bpb": 1.5})
    c = make("c")
    torch.manual_seed(999)                       # whatever the fresh process had drawn is overwritten by the file
    assert c.load_state(path) == {"min_bpb": 1.5}
    assert c.step == 3 and c.dupe_active == b.dupe_active
    losses_c = [c.train_step()["loss"] for _ in range(3)]
    assert losses_b + losses_c == losses_a
    for (n, p), (_, q) in zip(a.model.named_parameters(), c.model.named_parameters()):
        assert torch.equal(p, q), n
    sa, sc = a.optimizer.state_dict()["tensors"], c.optimizer.state_dict()["tensors"]
    assert all(torch.equal(sa[k], sc[k]) for k in sa)


def test_fit_writes_resume_files_and_picks_them_up(corpus, tmp_path):
    from slowrun_b200.train.trainer import Trainer
    cfg = _shrink(track_defaults("limited"), corpus, tmp_path)
    cfg.num_epochs, cfg.swa_last_epochs, cfg.logit_avg, cfg.dupe_start_epoch = 2, 0, 0, 99
    cfg.save_every, cfg.max_steps, cfg.resume = 2, 4, str(tmp_path / "r" / "state")
    Trainer(cfg, _info(), quiet=True).fit()
    assert os.path.exists(cfg.resume + ".rank0")
    cfg.max_steps = 6
    tr = Trainer(cfg, _info(), quiet=True)
    res = tr.fit()
    assert res["steps"] == 6 and tr.step == 6


def test_resume_replays_window_stages_and_restores_the_ema(corpus, tmp_path):
    """A run stopped in the second window stage of the two-hour track comes back with the long window, the rescaled rotary
    table and the softmax scale of that stage; a tiny-track run comes back with its weight EMA."""
    from slowrun_b200.train.trainer import Trainer
    cfg = _shrink(track_defaults("two_hour"), corpus, tmp_path / "a")
    cfg.num_epochs, cfg.swa_last_epochs, cfg.logit_avg, cfg.dupe_start_epoch = 3, 0, 0, 99
    cfg.window_schedule = "1-1:16,32;2-3:32,64"
    cfg.max_steps, cfg.save_every, cfg.resume = 1000, 0, None
    tr = Trainer(cfg, _info(), quiet=True)
    # run into epoch 2 through fit's own epoch handling
    cfg.max_steps = tr.sched.steps_per_epoch and int(tr.sched.steps_per_epoch) + 2
    tr.fit()
    assert tr.current_epoch == 2 and tr.model.long_window == 64 and tr.model.rotary.yarn_active
    path = str(tmp_path / "state" / "s")
    tr.save_state(path)
    want_cos, want_scale, want_step = tr.model.rotary.cos.clone(), tr.model.rotary.attn_scale, tr.step
    want_loss = tr.train_step()["loss"]            # the step the resumed run has to reproduce (dropout is on: same RNG stream)
    cfg2 = _shrink(track_defaults("two_hour"), corpus, tmp_path / "b")
    cfg2.num_epochs, cfg2.swa_last_epochs, cfg2.logit_avg, cfg2.dupe_start_epoch = 3, 0, 0, 99
    cfg2.window_schedule = cfg.window_schedule
    tr2 = Trainer(cfg2, _info(), quiet=True)
    assert tr2.model.long_window == 32 and not tr2.model.rotary.yarn_active
    tr2.load_state(path)
    assert tr2.step == want_step and tr2.current_epoch == 2 and tr2.model.long_window == 64
    assert tr2.model.rotary.attn_scale == want_scale
    assert torch.equal(tr2.model.rotary.cos, want_cos)
    assert tr2.train_step()["loss"] == want_loss

    tcfg = _shrink(track_defaults("tiny"), corpus, tmp_path / "t")
    tcfg.update_ema_every, tcfg.model.dropout = 1, 0.0
    tt = Trainer(tcfg, _info(), quiet=True)
    for _ in range(3):
        tt.train_step()
    tt.save_state(str(tmp_path / "state" / "t"))
    tcfg2 = _shrink(track_defaults("tiny"), corpus, tmp_path / "t2")
    tcfg2.update_ema_every, tcfg2.model.dropout = 1, 0.0
    tt2 = Trainer(tcfg2, _info(), quiet=True)
    tt2.load_state(str(tmp_path / "state" / "t"))
    assert tt2.ema.updates == tt.ema.updates == 3
    assert all(torch.equal(a, b) for a, b in zip(tt.ema.ema, tt2.ema.ema))
