"""Universal transformer at the "unlimited" size: 48 shared-weight layers of width 4096, 131 072-token batches, and a
separate `mtp_head` that predicts the token after next from the final hidden state (weight 0.3)
(research/universal_transformer/train_unlimited.py:38-77, 367-369, 598-604). Same trainer and flags as `train.py`
beside this file, plus `--mtp-weight`.

    torchrun --standalone --nproc_per_node=8 research/universal_transformer/train_unlimited.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import train as _ut  # noqa: E402

DEFAULTS = dict(device_batch_size=1, weight_decay=0.65, total_batch_size=131072, schedule="0:48", n_head=32, n_embd=4096,
                lr_multiplier=0.125, mtp_weight=0.3)

if __name__ == "__main__":
    _ut.main(defaults=DEFAULTS)
