"""Loss-curve parity: the unmodified reference script and this framework on the same synthetic corpus, same seed,
same flags, dropout and stochastic depth off (their random streams differ by construction), one GPU.

    python baseline/loss_parity.py [--track limited|tiny] [--n_layer 8 --n_embd 512 --n_head 4 --steps 20 --total-batch-size 32768]

Each arm runs in its own process. The reference arm goes through `ref_runner` (stand-ins for tiktoken / wandb / the
attention loader only) and its curve is what the script itself hands to `wandb_run.log` as "train/loss" (the
debiased 0.9-EMA of the last micro-batch loss, train.py:1193-1204). Our arm computes the same statistic from
`Trainer.train_step()`. Prints one JSON line: both curves and the largest absolute difference.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)


def flags(a):
    f = ["--n_layer", str(a.n_layer), "--n_embd", str(a.n_embd), "--n_head", str(a.n_head), "--device-batch-size",
         str(a.device_batch_size), "--total-batch-size", str(a.total_batch_size), "--dropout", "0"]
    return f + (["--stoch-depth", "0"] if a.track == "limited" else [])      # the tiny script has no stochastic depth


def arm_reference(a, data_dir):
    import ref_runner
    res = ref_runner.run(a.track, a.steps, 0, flags(a) + ["--run-name", "parity_ref"], data_dir,
                         os.path.join(tempfile.gettempdir(), "slowrun_parity_work"))
    return [float(e["train/loss"]) for e in res["wandb_log"] if "train/loss" in e][:a.steps]


def arm_ours(a, data_dir):
    from slowrun_b200.config import config_from_args
    from slowrun_b200.train.trainer import Trainer
    argv = flags(a) + ["--input_bin", os.path.join(data_dir, "fineweb_train.pt"), "--input_val_bin",
                       os.path.join(data_dir, "fineweb_val.pt")]
    cfg = config_from_args(a.track, argv)
    if a.bf16_head:
        cfg.model.fp8_lm_head = False      # noise floor of the fp8 head: the same run with bf16 operands in the loss head
    tr = Trainer(cfg, quiet=True)
    out, smooth = [], 0.0
    for k in range(1, a.steps + 1):
        loss = tr.train_step(sync=True)["loss"]
        smooth = 0.9 * smooth + 0.1 * loss
        out.append(smooth / (1 - 0.9 ** k))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--arm", default="both", choices=["both", "reference", "ours"])
    ap.add_argument("--track", default="limited", choices=["limited", "tiny"])
    ap.add_argument("--bf16-head", action="store_true",
                    help="tiny: add a third curve, this framework with a bf16 loss head (how far fp8 rounding alone moves the curve)")
    ap.add_argument("--n_layer", type=int, default=8)
    ap.add_argument("--n_embd", type=int, default=512)
    ap.add_argument("--n_head", type=int, default=4)
    ap.add_argument("--device-batch-size", type=int, default=4)
    ap.add_argument("--total-batch-size", type=int, default=32768)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--data-dir", default=None)
    a = ap.parse_args()
    data_dir = a.data_dir or os.path.join(tempfile.gettempdir(), f"slowrun_parity_{a.total_batch_size}_{a.steps}")
    if not os.path.exists(os.path.join(data_dir, "fineweb_train.pt")):
        from slowrun_b200.data.synthetic import write_synthetic_corpus
        write_synthetic_corpus(data_dir, train_tokens=(a.steps + 4) * a.total_batch_size + 2049 * 64, val_tokens=1_100_000)
    if a.arm != "both":
        curve = arm_reference(a, data_dir) if a.arm == "reference" else arm_ours(a, data_dir)
        print("CURVE " + json.dumps(curve), flush=True)
        return
    curves = {}
    for arm in ("reference", "ours"):
        cmd = [sys.executable, os.path.abspath(__file__), "--arm", arm, "--track", a.track, "--data-dir", data_dir] + \
              [x for kv in (("--n_layer", a.n_layer), ("--n_embd", a.n_embd), ("--n_head", a.n_head),
                            ("--device-batch-size", a.device_batch_size), ("--total-batch-size", a.total_batch_size),
                            ("--steps", a.steps)) for x in (kv[0], str(kv[1]))]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
        line = [ln for ln in r.stdout.splitlines() if ln.startswith("CURVE ")]
        if not line:
            print(json.dumps({"arm": arm, "failed": (r.stderr or r.stdout)[-600:]}))
            return
        curves[arm] = json.loads(line[-1][6:])
    if a.bf16_head:
        cmd = [sys.executable, os.path.abspath(__file__), "--arm", "ours", "--bf16-head", "--track", a.track, "--data-dir", data_dir] + \
              [x for kv in (("--n_layer", a.n_layer), ("--n_embd", a.n_embd), ("--n_head", a.n_head),
                            ("--device-batch-size", a.device_batch_size), ("--total-batch-size", a.total_batch_size),
                            ("--steps", a.steps)) for x in (kv[0], str(kv[1]))]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
        line = [ln for ln in r.stdout.splitlines() if ln.startswith("CURVE ")]
        curves["ours_bf16_head"] = json.loads(line[-1][6:]) if line else None
    n = min(len(curves["reference"]), len(curves["ours"]))
    diff = [abs(curves["reference"][i] - curves["ours"][i]) for i in range(n)]
    print(json.dumps({"what": "loss_parity", "config": vars(a), "reference": curves["reference"], "ours": curves["ours"],
                      "ours_bf16_head": curves.get("ours_bf16_head"), "max_abs_diff": max(diff) if diff else None, "steps_compared": n}))


if __name__ == "__main__":
    main()
