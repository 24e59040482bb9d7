"""Validation: bits-per-byte and mean loss, and the probability-averaged checkpoint ensemble.

`evaluate_bpb` computes what train.py:846-873 computes, `evaluate_prob_avg` what train.py:876-941 computes
(checkpoint-outer, batch-inner; accumulates w * p(target) and scores -log of the mixture). The token-byte table of the reference comes
from tiktoken (train.py:1027-1038); without network access `default_token_bytes` substitutes a fixed table, which
changes BPB's denominator but not the loss.
"""
from __future__ import annotations

import math

import torch

from ..config import VOCAB_SIZE, BOS_ID


def default_token_bytes(device, vocab_size: int = VOCAB_SIZE) -> torch.Tensor:
    """tiktoken's gpt2 byte lengths when the package and its cached vocabulary are available, else a deterministic
    stand-in (BOS = 0 bytes, others 1 + id % 7)."""
    try:
        import tiktoken
        enc = tiktoken.get_encoding("gpt2")
        eot = enc._special_tokens["<|endoftext|>"]
        tb = [0 if i == eot else len(enc.decode_single_token_bytes(i)) for i in range(enc.n_vocab)]
    except Exception:
        tb = [0 if i == BOS_ID else 1 + (i % 7) for i in range(vocab_size)]
    return torch.tensor(tb, dtype=torch.int32, device=device)


class _Tally:
    """Running sums behind both metrics: nats over tokens that have bytes, bytes, nats over scored tokens, scored
    tokens. They stay on the device in one fp64 vector, so a rank contributes with a single all-reduce at the end
    (the reference issues four, train.py:865-868)."""

    def __init__(self, device, token_bytes):
        self.sums = torch.zeros(4, dtype=torch.float64, device=device)
        self.token_bytes = token_bytes

    def add(self, nats: torch.Tensor, targets: torch.Tensor):
        """nats: fp32 per-token -log p(target) (any value where the target is -1); targets: same shape, int64."""
        nats, y = nats.reshape(-1), targets.reshape(-1)
        scored = y >= 0
        nbytes = self.token_bytes[y.clamp_min(0)] * scored        # an ignored position has neither bytes nor nats
        has_bytes = nbytes > 0
        self.sums += torch.stack([(nats * has_bytes).sum(), nbytes.sum(), (nats * scored).sum(), scored.sum()]).double()

    def result(self, comm=None):
        if comm is not None:
            comm.all_reduce_sum(self.sums, async_op=False)
        nats, nbytes, loss, ntok = self.sums.tolist()
        bpb = nats / (math.log(2) * nbytes) if nbytes > 0 else float("inf")
        return bpb, (loss / ntok if ntok > 0 else float("inf"))


@torch.no_grad()
def evaluate_bpb(model, batches, steps, token_bytes, comm=None, num_iterations=None):
    """(bits per byte, mean loss) over `steps` batches of `batches` (train.py:846-873)."""
    tally = _Tally(model.get_device(), token_bytes)
    it = iter(batches)
    kw = {} if num_iterations is None else {"num_iterations": num_iterations}
    for _ in range(steps):
        x, y, _ = next(it)
        tally.add(model(x, y, loss_reduction="none", **kw).float(), y)
    return tally.result(comm)


@torch.no_grad()
def evaluate_prob_avg(model, build_val_loader, ckpt_paths, weights, steps, token_bytes, comm=None, load_fn=None):
    """Mixture-of-checkpoints evaluation (train.py:876-941): p(y_t) = sum_c w_c p_c(y_t), scored as
    -log max(p, 1e-40).

    Each member's p(y_t) comes from the per-token loss the head kernel already produces (p = exp(-loss)), so no
    [tokens, vocab] softmax is ever materialised; what is kept across checkpoints is one fp32 value per token."""
    from .checkpoint import load_named_params
    dev = model.get_device()
    loader = build_val_loader()
    batches = []
    for _ in range(steps):
        x, y, _ = next(loader)
        batches.append((x, y))
    mix = [torch.zeros(y.numel(), dtype=torch.float32, device=dev) for _, y in batches]
    for path, w in zip(ckpt_paths, weights):
        (load_fn or load_named_params)(model, torch.load(path, map_location="cpu", weights_only=True))
        for (x, y), m in zip(batches, mix):
            nll = model(x, y, loss_reduction="none").reshape(-1).float()
            m.add_(torch.exp(-nll) * (y.reshape(-1) >= 0), alpha=float(w))
    tally = _Tally(dev, token_bytes)
    for (_, y), m in zip(batches, mix):
        tally.add(-torch.log(m.clamp_min(1e-40)), y)
    return tally.result(comm)
