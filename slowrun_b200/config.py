"""Typed per-track configuration and the argparse bridge.

Every flag of the reference's four entry points is accepted with its original spelling and default
(limited: train.py:40-95, tiny: tiny/train.py:55-129, two-hour: two_hour/train.py:39-93,
unlimited: unlimited/train.py:74-187). The reference freezes the values into module globals; here they
become one `TrainConfig` dataclass that model, optimizer and loop read explicitly.
"""
from __future__ import annotations

import argparse
from dataclasses import dataclass, field, asdict
from typing import Optional, Sequence

TRACKS = ("limited", "tiny", "two_hour", "unlimited")

MAX_SEQ_LEN = 2048
WINDOW_PATTERN = "SSSL"
EVAL_TOKENS = 10_000_000
BOS_ID = 50256
VOCAB_SIZE = 50257
ADAM_BETAS = (0.8, 0.95)


@dataclass
class ModelConfig:
    """Architecture switches of the GPT family. Defaults are the limited track's (train.py:221-233)."""
    sequence_len: int = MAX_SEQ_LEN
    vocab_size: int = VOCAB_SIZE
    n_layer: int = 30
    n_head: int = 14
    n_kv_head: int = 14
    n_embd: int = 1792
    window_pattern: str = WINDOW_PATTERN
    dropout: float = 0.1
    mlp_dropout: bool = True          # tiny applies dropout to the attention output only
    stoch_depth: float = 0.05
    use_iha: bool = True
    iha_mix_v: bool = True
    logit_cap: float = 10.0
    mtp_weight: float = 0.3           # extra-block MTP (limited / two-hour / unlimited); 0 = off
    # tiny-track features
    xsa_mode: str = "off"             # off | first6 | all
    xsa_eps: float = 1e-4
    key_offset: bool = False          # partial key offset on long-window layers
    rope_truncate: bool = False       # half-truncated RoPE
    num_iterations: int = 1           # whole-network recurrence (tiny)
    fused_mtp: bool = False           # shared-head shifted-target MTP through the fused CE (tiny)
    lm_head_transposed: bool = False  # tiny stores lm_head as (n_embd, vocab) bf16
    resid_lambda_init: float = 1.0
    cproj_zero_init: bool = False
    attn_gate_adamw: bool = False     # tiny steps attn_gate with AdamW; the other tracks hand it to Muon
    fp8_lm_head: bool = False         # e4m3 operands for the lm-head forward product of the training loss (tiny track)
    mlp_hidden: Optional[int] = None  # override; default 256*ceil((8d/3)/256)
    label_smoothing: float = 0.0      # unlimited

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def padded_vocab(self) -> int:
        return ((self.vocab_size + 63) // 64) * 64

    @property
    def hidden(self) -> int:
        if self.mlp_hidden is not None:
            return self.mlp_hidden
        return 256 * ((8 * self.n_embd // 3 + 255) // 256)


@dataclass
class TrainConfig:
    track: str = "limited"
    model: ModelConfig = field(default_factory=ModelConfig)
    device_batch_size: int = 4
    num_epochs: int = 11
    patience: int = -1
    run_name: Optional[str] = None
    scalar_lr: float = 0.1
    matrix_lr: float = 0.04
    embedding_lr: float = 0.15
    unembedding_lr: float = 0.002
    lr_multiplier: float = 0.25
    weight_decay: float = 1.3
    total_batch_size: int = 524288
    warmup_ratio: float = 0.0
    warmdown_ratio: float = 0.2
    warmdown_power: float = 0.5       # limited: sqrt-shaped; tiny: 1.0 (linear)
    final_lr_frac: float = 0.0
    save_result: str = ""
    input_bin: Optional[str] = None
    input_val_bin: Optional[str] = None
    wandb_group: Optional[str] = None
    dupe_start_epoch: int = 7
    dupe_layers_start: int = 15
    dupe_layers_end: int = 21
    dupe_loops: int = 2
    logit_avg: int = 3
    logit_avg_dir: str = "logit_avg_ckpts"
    logit_avg_mode: str = "both"
    eval_logit_avg: bool = False
    swa_last_epochs: int = 3
    iha_lr: float = 0.02
    no_doc_shuffle: bool = False
    # WD schedule (limited/two-hour constants, train.py:137-139)
    wd_pre_hold_frac: float = 0.40
    wd_swa_low: float = 0.65
    wd_swa_high: float = 1.50
    # tiny-only
    wd_phase1_epoch: float = 2.0
    wd_phase2_epoch: float = 8.0
    wd_mid: float = 0.1
    wd_end: float = 0.93
    iteration_schedule: str = "late-transition"
    min_iterations: int = 1
    iteration_transition_ratio: float = 0.3
    update_ema_every: int = 10
    ema_decay_per_epoch: float = 0.15
    max_train_steps: int = 3040
    mtp_predict: int = 3
    mtp_anneal_frac: float = 0.66
    # two-hour only
    window_schedule: str = ""
    # unlimited only
    num_models: int = 480
    epochs_per_cycle: float = 2.0
    seed: int = 42
    gpus_per_node: int = 8
    checkpoint_base: str = "checkpoints"
    resume: Optional[str] = None
    adam_betas: Sequence[float] = ADAM_BETAS
    muon_momentum: float = 0.95
    ns_steps: int = 5
    pgt_steps: int = 16
    distill_alpha: float = 0.45
    distill_temperature: float = 1.2
    distill_after_cycles: int = 8
    perturb_scale: float = 0.25
    perturb_scale_min: float = 0.05
    fitness_tokens: int = 132000
    grad_opt_steps: int = 300
    grad_lr: float = 0.5
    grad_weighted_eval: bool = False
    k_sweep: Sequence[int] = (8, 16, 32, 64, 128, 256)
    lr_floor: float = 0.08
    wd_schedule: str = "inverse_lr"
    wd_floor: float = 0.7
    bs_schedule: str = "triangular"
    bs_floor: int = 393216
    dupe_after_n_models: int = 0
    # framework switches (no counterpart in the reference)
    comm: str = "auto"                # auto | fused | nccl : gradient/param collectives
    wire_dtype: str = "bf16"          # bf16 | fp32 : gradient reduce-scatter wire format
    cuda_graphs: bool = True          # replay each micro-batch's forward+backward as one captured CUDA graph
    max_steps: int = -1               # stop after this many optimizer steps (benchmarks/tests)
    overlap_backward: bool = False    # pull each layer's gradients to their owners while the last backward pass still runs
    save_every: int = 0               # write a resume file (--resume PATH, default <run dir>/resume) every N optimizer steps
    eval_tokens: int = EVAL_TOKENS
    log_jsonl: str = ""
    wandb: bool = False
    runs_dir: str = "runs"
    data_dir: str = "fineweb_data"

    def to_dict(self):
        return asdict(self)

    # derived learning rates (train.py:124-129)
    @property
    def lrs(self):
        m = self.lr_multiplier if self.lr_multiplier is not None else 1.0
        return dict(matrix=self.matrix_lr * m, unembedding=self.unembedding_lr * m,
                    embedding=self.embedding_lr * m, scalar=self.scalar_lr * m)


def track_defaults(track: str) -> TrainConfig:
    """Defaults of each reference entry point."""
    if track == "limited":
        return TrainConfig(track="limited")
    if track == "two_hour":
        return TrainConfig(track="two_hour", num_epochs=22, dupe_start_epoch=14, logit_avg=11, swa_last_epochs=8,
                           window_schedule="1-6:256,768;7-13:768,1792;14-22:1280,2048")
    if track == "tiny":
        m = ModelConfig(n_layer=16, n_head=8, n_kv_head=8, n_embd=1024, dropout=0.1, mlp_dropout=False,
                        stoch_depth=0.0, use_iha=False, iha_mix_v=False, logit_cap=15.0, mtp_weight=0.0,
                        xsa_mode="all", key_offset=True, rope_truncate=True, num_iterations=2, fused_mtp=True,
                        lm_head_transposed=True, resid_lambda_init=1.1, cproj_zero_init=True, fp8_lm_head=True,
                        attn_gate_adamw=True)
        return TrainConfig(track="tiny", model=m, device_batch_size=32, num_epochs=15, scalar_lr=0.25,
                           unembedding_lr=0.001, lr_multiplier=0.8, weight_decay=0.8, warmdown_ratio=0.4,
                           warmdown_power=1.0, swa_last_epochs=4, logit_avg=0, dupe_start_epoch=10 ** 9)
    if track == "unlimited":
        m = ModelConfig(n_layer=30, n_head=16, n_kv_head=16, n_embd=2048, stoch_depth=0.0, logit_cap=15.0)
        return TrainConfig(track="unlimited", model=m, device_batch_size=2, dupe_layers_end=25, dupe_loops=4,
                           dupe_start_epoch=0, logit_avg=0, swa_last_epochs=0)
    raise ValueError(f"unknown track {track!r}")


def build_parser(track: str) -> argparse.ArgumentParser:
    d = track_defaults(track)
    m = d.model
    p = argparse.ArgumentParser(description=f"slowrun_b200 {track} track")
    a = p.add_argument
    a("--device-batch-size", type=int, default=d.device_batch_size)
    a("--scalar-lr", type=float, default=d.scalar_lr)
    a("--matrix-lr", type=float, default=d.matrix_lr)
    a("--weight-decay", type=float, default=d.weight_decay)
    a("--total-batch-size", type=int, default=d.total_batch_size)
    a("--save-result", type=str, default="")
    a("--n_layer", type=int, default=m.n_layer)
    a("--n_head", type=int, default=m.n_head)
    a("--n_embd", type=int, default=m.n_embd)
    a("--lr_multiplier", type=float, default=d.lr_multiplier)
    a("--input_bin", type=str, default=None)
    a("--input_val_bin", type=str, default=None)
    a("--output_json", type=str, default=None)
    a("--wandb_group", type=str, default=None)
    a("--dropout", type=float, default=m.dropout)
    a("--no-doc-shuffle", action="store_true")
    a("--warmdown-ratio", type=float, default=None)
    if track in ("limited", "tiny", "two_hour"):
        a("--num-epochs", type=int, default=d.num_epochs)
        a("--patience", type=int, default=-1)
        a("--swa-last-epochs", type=int, default=d.swa_last_epochs)
    if track in ("limited", "tiny"):
        a("--run-name", type=str, default=None)
    else:
        a("--run", type=str, default=None, dest="run_name")
    if track in ("limited", "two_hour"):
        a("--dupe-start-epoch", type=int, default=d.dupe_start_epoch)
        a("--dupe-layers-start", type=int, default=d.dupe_layers_start)
        a("--dupe-layers-end", type=int, default=d.dupe_layers_end)
        a("--dupe-loops", type=int, default=d.dupe_loops)
        a("--logit-cap", type=float, default=m.logit_cap)
        a("--logit-avg", type=int, default=d.logit_avg)
        a("--logit-avg-dir", type=str, default=d.logit_avg_dir)
        a("--logit-avg-mode", type=str, default="both", choices=["equal", "weighted", "both"])
        a("--eval-logit-avg", action="store_true")
        a("--stoch-depth", type=float, default=m.stoch_depth)
    if track in ("limited", "two_hour", "unlimited"):
        a("--mtp-weight", type=float, default=m.mtp_weight)
        a("--iha", action="store_true", default=True)
        a("--no-iha", action="store_false", dest="iha")
        a("--iha-lr", type=float, default=d.iha_lr)
    if track == "two_hour":
        a("--window-schedule", type=str, default=d.window_schedule)
    if track in ("tiny", "unlimited"):
        a("--embedding-lr", type=float, default=d.embedding_lr)
        a("--unembedding-lr", type=float, default=d.unembedding_lr)
    if track == "tiny":
        a("--warmup-ratio", type=float, default=0.0)
        a("--wd-phase1-epoch", type=float, default=d.wd_phase1_epoch)
        a("--wd-phase2-epoch", type=float, default=d.wd_phase2_epoch)
        a("--wd-mid", type=float, default=d.wd_mid)
        a("--wd-end", type=float, default=d.wd_end)
        a("--num-iterations", type=int, default=m.num_iterations)
        a("--iteration-schedule", type=str, default=d.iteration_schedule, choices=["constant", "late-transition"])
        a("--min-iterations", type=int, default=d.min_iterations)
        a("--iteration-transition-ratio", type=float, default=d.iteration_transition_ratio)
        a("--update-ema-every", type=int, default=d.update_ema_every)
        a("--ema-decay-per-epoch", type=float, default=d.ema_decay_per_epoch)
        a("--max-train-steps", type=int, default=d.max_train_steps)
        a("--xsa-mode", type=str, default=m.xsa_mode, choices=["off", "first6", "all"])
        a("--mtp-predict", type=int, default=d.mtp_predict)
        a("--mtp-anneal-frac", type=float, default=d.mtp_anneal_frac)
    if track == "unlimited":
        a("--num-models", type=int, default=d.num_models)
        a("--epochs-per-cycle", type=float, default=d.epochs_per_cycle)
        a("--seed", type=int, default=d.seed)
        a("--gpus-per-node", type=int, default=d.gpus_per_node)
        a("--checkpoint-base", type=str, default=d.checkpoint_base)
        a("--resume", type=str, default=None)
        a("--label-smoothing", type=float, default=0.0)
        a("--adam-betas", type=float, nargs=2, default=list(ADAM_BETAS))
        a("--muon-momentum", type=float, default=d.muon_momentum)
        a("--ns-steps", type=int, default=d.ns_steps)
        a("--pgt-steps", type=int, default=d.pgt_steps)
        a("--distill-alpha", type=float, default=d.distill_alpha)
        a("--distill-temperature", type=float, default=d.distill_temperature)
        a("--distill-after-cycles", type=int, default=d.distill_after_cycles)
        a("--perturb-scale", type=float, default=d.perturb_scale)
        a("--perturb-scale-min", type=float, default=d.perturb_scale_min)
        a("--fitness-tokens", type=int, default=d.fitness_tokens)
        a("--grad-opt-steps", type=int, default=d.grad_opt_steps)
        a("--grad-lr", type=float, default=d.grad_lr)
        a("--grad-weighted-eval", action="store_true")
        a("--k-sweep", type=int, nargs="+", default=list(d.k_sweep))
        a("--lr-floor", type=float, default=d.lr_floor)
        a("--wd-schedule", type=str, default=d.wd_schedule)
        a("--wd-floor", type=float, default=d.wd_floor)
        a("--bs-schedule", type=str, default=d.bs_schedule)
        a("--bs-floor", type=int, default=d.bs_floor)
        a("--dupe-after-n-models", type=int, default=0)
        a("--dupe-layers-start", type=int, default=d.dupe_layers_start)
        a("--dupe-layers-end", type=int, default=d.dupe_layers_end)
    # framework switches
    a("--comm", type=str, default="auto", choices=["auto", "fused", "nccl"])
    a("--wire-dtype", type=str, default="bf16", choices=["bf16", "fp32"])
    a("--overlap-backward", action="store_true", help="peer-memory optimizer: gradient pulls under the last backward pass")
    a("--no-cuda-graphs", action="store_false", dest="cuda_graphs")
    a("--max-steps", type=int, default=-1)
    if track != "unlimited":
        a("--resume", type=str, default=None, help="path prefix of the resume files (<prefix>.rank<r>); continue from them if present")
        a("--save-every", type=int, default=0, help="write the resume files every N optimizer steps")
    a("--eval-tokens", type=int, default=EVAL_TOKENS)
    a("--log-jsonl", type=str, default="")
    a("--wandb", action="store_true")
    return p


def config_from_args(track: str, argv=None) -> TrainConfig:
    ns = build_parser(track).parse_args(argv)
    cfg = track_defaults(track)
    m = cfg.model
    v = vars(ns)
    for key, val in v.items():
        if key in ("n_layer", "n_head", "n_embd", "dropout"):
            setattr(m, key, val)
        elif key == "stoch_depth":
            m.stoch_depth = val
        elif key == "logit_cap":
            m.logit_cap = val
        elif key == "mtp_weight":
            m.mtp_weight = val
        elif key == "iha":
            m.use_iha = val
            m.iha_mix_v = val
        elif key == "xsa_mode":
            m.xsa_mode = val
        elif key == "num_iterations":
            m.num_iterations = val
        elif key == "label_smoothing":
            m.label_smoothing = val
        elif key == "warmdown_ratio":
            if val is not None:
                cfg.warmdown_ratio = val
        elif key == "output_json":
            pass
        elif hasattr(cfg, key):
            setattr(cfg, key, val)
    m.n_kv_head = m.n_head
    if ns.output_json and not cfg.save_result:
        cfg.save_result = ns.output_json
    if track == "unlimited":
        m.mtp_weight = v.get("mtp_weight", m.mtp_weight)
    return cfg
