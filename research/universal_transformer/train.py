"""Universal transformer: attention and MLP weights shared across depth, per-layer norms and gates, and an active depth
that grows during training (`--n-layer-schedule "0:10,1533:20"`: 10 layers from step 0, 20 from step 1533).

    torchrun --standalone --nproc_per_node=8 research/universal_transformer/train.py

Accepts the flags of the reference script of the same name (research/universal_transformer/train.py:38-77).
`train_unlimited.py` beside this file is the same trainer with the larger defaults and the separate `mtp_head` of
research/universal_transformer/train_unlimited.py.
"""
import argparse
import os
import sys

os.environ.setdefault("PYTORCH_ALLOC_CONF", "expandable_segments:True")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from slowrun_b200.config import track_defaults  # noqa: E402
from slowrun_b200.models.research import UniversalConfig, parse_depth_schedule  # noqa: E402
from slowrun_b200.parallel.comm import shutdown  # noqa: E402
from slowrun_b200.train.research import UniversalTrainer  # noqa: E402

DEFAULTS = dict(device_batch_size=4, weight_decay=0.8, total_batch_size=524288, schedule="0:10,1533:20", n_head=16,
                n_embd=2048, lr_multiplier=0.25, mtp_weight=None)


def build_parser(d=DEFAULTS):
    p = argparse.ArgumentParser(description="universal-transformer research fork")
    a = p.add_argument
    a("--device-batch-size", type=int, default=d["device_batch_size"])
    a("--num-epochs", type=int, default=12)
    a("--patience", type=int, default=-1)
    a("--run", type=str, default=None)
    a("--scalar-lr", type=float, default=0.1)
    a("--matrix-lr", type=float, default=0.04)
    a("--weight-decay", type=float, default=d["weight_decay"])
    a("--total-batch-size", type=int, default=d["total_batch_size"])
    a("--save-result", type=str, default="")
    a("--n-layer-schedule", type=str, default=d["schedule"])
    a("--n_head", type=int, default=d["n_head"])
    a("--n_embd", type=int, default=d["n_embd"])
    a("--lr_multiplier", type=float, default=d["lr_multiplier"])
    a("--input_bin", type=str, default=None)
    a("--input_val_bin", type=str, default=None)
    a("--output_json", type=str, default=None)
    a("--wandb_group", type=str, default=None)
    a("--dropout", type=float, default=0.1)
    a("--stoch-depth", type=float, default=0.05)
    a("--warmdown-ratio", type=float, default=None)
    a("--logit-cap", type=float, default=10.0)
    a("--logit-avg", type=int, default=3)
    a("--logit-avg-dir", type=str, default="logit_avg_ckpts")
    a("--logit-avg-mode", type=str, default="both", choices=["equal", "weighted", "both"])
    a("--eval-logit-avg", action="store_true")
    a("--iha", action="store_true", default=True)
    a("--no-iha", action="store_false", dest="iha")
    a("--iha-lr", type=float, default=0.02)
    if d["mtp_weight"] is not None:
        a("--mtp-weight", type=float, default=d["mtp_weight"])
    a("--no-doc-shuffle", action="store_true")
    a("--max-steps", type=int, default=-1)
    a("--eval-tokens", type=int, default=None)
    a("--sequence-len", type=int, default=2048)
    return p


def configs_from(args):
    schedule = parse_depth_schedule(args.n_layer_schedule)
    max_depth = max(dd for _, dd in schedule)
    uc = UniversalConfig(sequence_len=args.sequence_len, n_layer=max_depth, n_head=args.n_head, n_embd=args.n_embd,
                         dropout=args.dropout, stoch_depth=args.stoch_depth, logit_cap=args.logit_cap,
                         depth_schedule=args.n_layer_schedule, use_iha=args.iha, iha_mix_v=args.iha,
                         mtp_weight=float(getattr(args, "mtp_weight", 0.0) or 0.0))
    cfg = track_defaults("limited")
    m = cfg.model
    m.n_layer, m.n_head, m.n_kv_head, m.n_embd, m.sequence_len = max_depth, args.n_head, args.n_head, args.n_embd, args.sequence_len
    m.dropout, m.stoch_depth, m.use_iha, m.logit_cap = args.dropout, args.stoch_depth, args.iha, args.logit_cap
    cfg.device_batch_size, cfg.num_epochs, cfg.patience, cfg.run_name = args.device_batch_size, args.num_epochs, args.patience, args.run
    cfg.scalar_lr, cfg.matrix_lr, cfg.weight_decay, cfg.lr_multiplier = args.scalar_lr, args.matrix_lr, args.weight_decay, args.lr_multiplier
    cfg.total_batch_size, cfg.iha_lr = args.total_batch_size, args.iha_lr
    cfg.save_result = args.output_json or args.save_result
    cfg.input_bin, cfg.input_val_bin, cfg.wandb_group = args.input_bin, args.input_val_bin, args.wandb_group
    cfg.warmdown_ratio = 0.2 if args.warmdown_ratio is None else args.warmdown_ratio
    cfg.logit_avg, cfg.logit_avg_dir, cfg.logit_avg_mode, cfg.eval_logit_avg = (
        args.logit_avg, args.logit_avg_dir, args.logit_avg_mode, args.eval_logit_avg)
    cfg.dupe_start_epoch = 10 ** 9
    cfg.no_doc_shuffle, cfg.max_steps = args.no_doc_shuffle, args.max_steps
    if args.eval_tokens is not None:
        cfg.eval_tokens = args.eval_tokens
    return cfg, uc


def main(argv=None, defaults=DEFAULTS):
    args = build_parser(defaults).parse_args(argv)
    cfg, uc = configs_from(args)
    trainer = UniversalTrainer(cfg, uc)
    try:
        return trainer.fit()
    finally:
        shutdown()


if __name__ == "__main__":
    main()
