"""two_hour track entry point: `torchrun --standalone --nproc_per_node=8 two_hour/train.py` (also runs as plain `python two_hour/train.py` on
one GPU or on CPU). Accepts the flags of the reference script of the same name."""
import os
import sys

os.environ.setdefault("PYTORCH_ALLOC_CONF", "expandable_segments:True")
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)) + '/..')

from slowrun_b200.config import config_from_args  # noqa: E402
from slowrun_b200.parallel.comm import shutdown  # noqa: E402
from slowrun_b200.train.trainer import Trainer  # noqa: E402


def main(argv=None):
    cfg = config_from_args("two_hour", argv)
    trainer = Trainer(cfg)
    try:
        return trainer.fit()
    finally:
        shutdown()


if __name__ == "__main__":
    main()
