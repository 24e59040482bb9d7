"""unlimited track entry point: `torchrun --nnodes=N --nproc_per_node=8 unlimited/train.py --num-models M [--resume RUN]`
(also runs single-process). Accepts the flags of the reference script of the same name."""
import os
import sys

os.environ.setdefault("PYTORCH_ALLOC_CONF", "expandable_segments:True")
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from slowrun_b200.config import config_from_args  # noqa: E402
from slowrun_b200.parallel.comm import shutdown  # noqa: E402
from slowrun_b200.train.unlimited import UnlimitedTrainer  # noqa: E402


def main(argv=None):
    cfg = config_from_args("unlimited", argv)
    if cfg.resume and not cfg.run_name:
        cfg.run_name = cfg.resume
    trainer = UnlimitedTrainer(cfg)
    try:
        return trainer.run()
    finally:
        shutdown()


if __name__ == "__main__":
    main()
