"""Hybrid softmax / linear-attention GPT (Gated DeltaNet or Kimi Delta Attention on selected layers).

    torchrun --standalone --nproc_per_node=8 research/hybrid_attn/train.py --gdn-layers "1,3,5,7,9,11,13,16,18,20,22,24,26,28"
    python research/hybrid_attn/train.py --linear-attn-type kda --n_embd 1024 --n_head 8      # one GPU or CPU

Accepts the flags of the reference script of the same name (research/hybrid_attn/train.py:54-118).
"""
import argparse
import os
import sys

os.environ.setdefault("PYTORCH_ALLOC_CONF", "expandable_segments:True")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from slowrun_b200.config import track_defaults  # noqa: E402
from slowrun_b200.models.hybrid import HybridSpec, parse_linear_layers  # noqa: E402
from slowrun_b200.parallel.comm import shutdown  # noqa: E402
from slowrun_b200.train.research import HybridTrainer  # noqa: E402


def build_parser():
    p = argparse.ArgumentParser(description="hybrid softmax / linear-attention research fork")
    a = p.add_argument
    a("--device-batch-size", type=int, default=4)
    a("--num-epochs", type=int, default=12)
    a("--patience", type=int, default=-1)
    a("--run", type=str, default=None)
    a("--scalar-lr", type=float, default=0.1)
    a("--matrix-lr", type=float, default=0.04)
    a("--weight-decay", type=float, default=1.3)
    a("--total-batch-size", type=int, default=524288)
    a("--save-result", type=str, default="")
    a("--n_layer", type=int, default=30)
    a("--n_head", type=int, default=14)
    a("--n_embd", type=int, default=1792)
    a("--lr_multiplier", type=float, default=0.25)
    a("--input_bin", type=str, default=None)
    a("--input_val_bin", type=str, default=None)
    a("--output_json", type=str, default=None)
    a("--wandb_group", type=str, default=None)
    a("--dropout", type=float, default=0.1)
    a("--muon-eq-r", action="store_true", dest="muon_eq_r", default=True)
    a("--no-muon-eq-r", action="store_false", dest="muon_eq_r")
    a("--muon-ns-schedule", type=str, default="polar-express", choices=("polar-express", "deepseek-v4"))
    a("--dupe-start-epoch", type=int, default=7)
    a("--dupe-layers-start", type=int, default=15)
    a("--dupe-layers-end", type=int, default=21)
    a("--dupe-loops", type=int, default=2)
    a("--warmdown-ratio", type=float, default=None)
    a("--ema-decays", type=str, default="0.95")
    a("--ema-start-frac", type=float, default=0.90)
    a("--checkpoint-avg", type=int, default=0)
    a("--grad-clip", type=float, default=0.0)
    a("--logit-cap", type=float, default=10.0)
    a("--gdn-layers", type=str, default="auto")
    a("--gdn-head-dim-mode", type=str, default="param-matched", choices=("param-matched", "square"))
    a("--gdn-no-conv", action="store_true")
    a("--gdn-use-recurrent", action="store_true")
    a("--gdn-profile", action="store_true")
    a("--linear-attn-type", type=str, default="gdn", choices=("gdn", "kda"))
    a("--no-doc-shuffle", action="store_true")
    a("--max-steps", type=int, default=-1)
    a("--eval-tokens", type=int, default=None)
    a("--sequence-len", type=int, default=2048)
    return p


def config_from(args):
    cfg = track_defaults("limited")
    m = cfg.model
    m.n_layer, m.n_head, m.n_kv_head, m.n_embd, m.sequence_len = args.n_layer, args.n_head, args.n_head, args.n_embd, args.sequence_len
    m.dropout, m.stoch_depth, m.use_iha, m.iha_mix_v, m.mtp_weight = args.dropout, 0.0, False, False, 0.0
    m.logit_cap, m.cproj_zero_init = args.logit_cap, True
    cfg.device_batch_size, cfg.num_epochs, cfg.patience, cfg.run_name = args.device_batch_size, args.num_epochs, args.patience, args.run
    cfg.scalar_lr, cfg.matrix_lr, cfg.weight_decay, cfg.lr_multiplier = args.scalar_lr, args.matrix_lr, args.weight_decay, args.lr_multiplier
    cfg.total_batch_size = args.total_batch_size
    cfg.save_result = args.output_json or args.save_result
    cfg.input_bin, cfg.input_val_bin, cfg.wandb_group = args.input_bin, args.input_val_bin, args.wandb_group
    cfg.dupe_start_epoch, cfg.dupe_layers_start, cfg.dupe_layers_end, cfg.dupe_loops = (
        args.dupe_start_epoch, args.dupe_layers_start, args.dupe_layers_end, args.dupe_loops)
    cfg.warmdown_ratio = 0.2 if args.warmdown_ratio is None else args.warmdown_ratio
    cfg.warmdown_power, cfg.swa_last_epochs, cfg.logit_avg = 1.0, 0, 0      # linear warm-down, no cosine cycles, no disk ring
    cfg.wd_pre_hold_frac = 2.0                                              # constant weight decay
    cfg.no_doc_shuffle, cfg.max_steps = args.no_doc_shuffle, args.max_steps
    if args.eval_tokens is not None:
        cfg.eval_tokens = args.eval_tokens
    cfg.muon_eq_r, cfg.muon_ns_schedule = args.muon_eq_r, args.muon_ns_schedule
    if args.linear_attn_type != "gdn" and args.gdn_head_dim_mode != "param-matched":
        raise SystemExit("--gdn-head-dim-mode only applies to --linear-attn-type gdn")
    if args.linear_attn_type == "kda" and args.gdn_use_recurrent:
        raise SystemExit("--gdn-use-recurrent is only implemented for --linear-attn-type gdn")
    spec = HybridSpec(layers=parse_linear_layers(args.gdn_layers, args.n_layer), kind=args.linear_attn_type,
                      head_dim_mode=args.gdn_head_dim_mode, no_conv=args.gdn_no_conv, use_recurrent=args.gdn_use_recurrent,
                      profile=args.gdn_profile)
    return cfg, spec


def main(argv=None):
    args = build_parser().parse_args(argv)
    cfg, spec = config_from(args)
    decays = [float(d) for d in args.ema_decays.split(",") if d.strip()] if args.ema_decays else []
    trainer = HybridTrainer(cfg, spec, grad_clip=args.grad_clip, ema_decays=decays, ema_start_frac=args.ema_start_frac,
                            checkpoint_avg=args.checkpoint_avg)
    try:
        return trainer.fit()
    finally:
        shutdown()


if __name__ == "__main__":
    main()
