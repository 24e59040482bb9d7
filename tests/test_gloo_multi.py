"""Two-rank Gloo runs on CPU of the host-side multi-process logic:
* Trainer.fit() crosses an epoch boundary with the checkpoint ring on: rank 0 writes, every rank waits on the host
  barrier, the probability-averaging pass reads the files rank 0 wrote;
* the unlimited track's gradient all-reduce that starts during the backward pass gives bit-identical gradients to the
  plain all-reduce after it;
* per-node overrides change one node's configuration only."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _env(rank, world, port):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(2)


def _small(cfg, corpus, work):
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 4, 128, 4, 4, 64
    m.dropout, m.stoch_depth = 0.0, 0.0
    cfg.device_batch_size, cfg.total_batch_size = 2, 2 * 64 * 2 * 2
    cfg.input_bin, cfg.input_val_bin = corpus
    cfg.eval_tokens, cfg.runs_dir = 1024, os.path.join(work, "runs")
    cfg.logit_avg_dir = os.path.join(work, "ring")
    return cfg


def _fit_worker(rank, world, port, corpus, work):
    _env(rank, world, port)
    from slowrun_b200.config import track_defaults
    from slowrun_b200.parallel.comm import init_distributed, shutdown
    from slowrun_b200.train.trainer import Trainer
    info = init_distributed("cpu", timeout_s=120)
    cfg = _small(track_defaults("limited"), corpus, work)
    cfg.num_epochs, cfg.logit_avg, cfg.swa_last_epochs, cfg.dupe_start_epoch, cfg.run_name = 3, 2, 1, 2, "fit2"
    cfg.dupe_layers_start, cfg.dupe_layers_end = 2, 3
    res = Trainer(cfg, info, quiet=True).fit()
    torch.save(res, os.path.join(work, f"fit_r{rank}.pt"))
    shutdown()


@pytest.mark.timeout(900)
def test_fit_crosses_epoch_boundaries_with_checkpoints_on_two_ranks(tmp_path):
    from slowrun_b200.data.synthetic import write_synthetic_corpus
    corpus = write_synthetic_corpus(str(tmp_path / "data"), train_tokens=12_000, val_tokens=6_000)
    mp.spawn(_fit_worker, args=(2, _free_port(), corpus, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = (torch.load(tmp_path / f"fit_r{r}.pt") for r in (0, 1))
    assert r0["steps"] == r1["steps"] and r0["steps"] >= 3
    assert r0["best_val_loss"] == r1["best_val_loss"]            # both ranks evaluated the same checkpoints
    ring = sorted(os.listdir(tmp_path / "ring"))
    assert len(ring) == 2 and all(f.startswith("epoch_") for f in ring)


def _reduce_worker(rank, world, port, work):
    _env(rank, world, port)
    from slowrun_b200.config import track_defaults
    from slowrun_b200.models.gpt import build_model
    from slowrun_b200.parallel.comm import TorchComm, init_distributed, shutdown
    from slowrun_b200.train.unlimited import OverlappedAllReduce, allreduce_gradients
    init_distributed("cpu", timeout_s=120)
    cfg = track_defaults("unlimited")
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 4, 128, 4, 4, 64
    m.dropout = 0.0
    model = build_model(m, "cpu", seed=0)
    model.set_dupe_layers(2, 3, 1)                   # a replayed layer: its bucket must wait for the LAST visit
    comm = TorchComm()
    g = torch.Generator().manual_seed(10 + rank)
    idx = torch.randint(0, 50257, (2, 64), generator=g)
    out = {}
    fired = []
    for mode in ("plain", "overlapped"):
        model.zero_grad_arena()
        red = OverlappedAllReduce(model, comm) if mode == "overlapped" else None
        if red is not None:
            red.arm()
            inner = model.layer_done_hook
            model.layer_done_hook = lambda i: (fired.append((i, len(red.handles))), inner(i))[1]
        loss, _ = model(idx, idx)
        loss.backward()
        if red is not None:
            in_flight_before_finish = len(red.handles)
            red.finish()
        else:
            allreduce_gradients(model, comm)
        out[mode] = {n: (model.arena.head_grad if n == "lm_head.weight" else p.grad).clone() for n, p in model.named_parameters()}
    torch.save({"grads": out, "fired": fired, "early": in_flight_before_finish}, os.path.join(work, f"red_r{rank}.pt"))
    shutdown()


@pytest.mark.timeout(600)
def test_overlapped_gradient_allreduce_equals_the_plain_one(tmp_path):
    mp.spawn(_reduce_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    r0, r1 = (torch.load(tmp_path / f"red_r{r}.pt") for r in (0, 1))
    for n in r0["grads"]["plain"]:
        assert torch.equal(r0["grads"]["plain"][n], r0["grads"]["overlapped"][n]), n
        assert torch.equal(r0["grads"]["overlapped"][n], r1["grads"]["overlapped"][n]), n
    layers = [i for i, _ in r0["fired"]]
    assert layers == sorted(layers, reverse=True) and set(layers) == {0, 1, 2, 3, 4}     # 4 = the extra prediction block
    assert r0["early"] > 0, "no reduction was issued before the backward pass ended"


def test_node_overrides_apply_to_one_node_only():
    from slowrun_b200.config import track_defaults
    from slowrun_b200.train.unlimited import config_for_node
    cfg = track_defaults("unlimited")
    table = {1: {"distill_alpha": 0.4, "lr_floor": 0.1, "label_smoothing": 0.05, "warmdown_frac": 0.2}}
    a, b = config_for_node(cfg, 0, table), config_for_node(cfg, 1, table)
    assert a.distill_alpha == cfg.distill_alpha and a.model.label_smoothing == 0.0
    assert b.distill_alpha == 0.4 and b.lr_floor == 0.1 and b.model.label_smoothing == 0.05 and b.cycle_warmdown_frac == 0.2
    assert b.node_overrides == {"1": table[1]} and cfg.distill_alpha != 0.4
    with pytest.raises(KeyError):
        config_for_node(cfg, 0, {0: {"no_such_option": 1}})


def _unlimited_worker(rank, world, port, corpus, work):
    _env(rank, world, port)
    from slowrun_b200.config import track_defaults
    from slowrun_b200.parallel.comm import init_distributed, shutdown
    from slowrun_b200.train.unlimited import UnlimitedTrainer
    info = init_distributed("cpu", timeout_s=300)
    cfg = _small(track_defaults("unlimited"), corpus, work)
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head = 2, 64, 2, 2
    cfg.gpus_per_node = 2                                   # 4 ranks = 2 nodes of 2: two chains of 2 snapshots each
    cfg.total_batch_size = 2 * 64 * 2
    cfg.num_models, cfg.epochs_per_cycle, cfg.distill_after_cycles = 4, 0.1, 1
    cfg.bs_floor = cfg.total_batch_size
    cfg.fitness_tokens, cfg.pgt_steps, cfg.k_sweep, cfg.grad_opt_steps = 1000, 2, (2, 4), 20
    cfg.checkpoint_base, cfg.run_name = os.path.join(work, "ck"), "u"
    cfg.dupe_layers_start, cfg.dupe_layers_end, cfg.dupe_loops = 1, 2, 1
    tr = UnlimitedTrainer(cfg, info, node_overrides={1: {"matrix_lr": cfg.matrix_lr * 0.5}})
    out = tr.run()
    torch.save({"node": tr.node_rank, "leader": tr.is_leader, "indices": tr.model_indices, "matrix_lr": tr.cfg.matrix_lr,
                "models": out["models"], "ensemble": out["ensemble"], "selection": out["selection"]},
               os.path.join(work, f"unl_r{rank}.pt"))
    shutdown()


@pytest.mark.timeout(1200)
def test_unlimited_chains_on_two_nodes_meet_for_selection_and_ensemble(tmp_path):
    """Ensemble training across nodes (unlimited/train.py:1870-1960, 2160-2290): each node trains its own chain with
    data parallelism inside the node; all ranks then share the target probabilities, run the greedy selection and
    evaluate the mixtures with the members dealt over every rank."""
    from slowrun_b200.data.synthetic import write_synthetic_corpus
    corpus = write_synthetic_corpus(str(tmp_path / "data"), train_tokens=12_000, val_tokens=6_000)
    mp.spawn(_unlimited_worker, args=(4, _free_port(), corpus, str(tmp_path)), nprocs=4, join=True)
    res = [torch.load(tmp_path / f"unl_r{r}.pt", weights_only=False) for r in range(4)]
    assert [r["node"] for r in res] == [0, 0, 1, 1] and [r["leader"] for r in res] == [True, False, True, False]
    assert res[0]["indices"] == [0, 1] and res[2]["indices"] == [2, 3]
    assert res[2]["matrix_lr"] == pytest.approx(res[0]["matrix_lr"] * 0.5)          # per-node override
    assert all(os.path.exists(tmp_path / "ck" / "u" / f"model_{i}.pt") for i in range(4))
    for r in res[1:]:                                        # every rank ends with the same selection and the same numbers
        assert r["selection"] == res[0]["selection"]
        assert r["ensemble"] == res[0]["ensemble"]
    assert set(res[0]["ensemble"]) == {2, 4} and res[0]["ensemble"][4]["val_loss"] < 11.0
