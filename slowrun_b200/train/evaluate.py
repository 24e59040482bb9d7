"""Validation: bits-per-byte and mean loss, and the probability-averaged checkpoint ensemble.

`evaluate_bpb` follows train.py:846-873, `evaluate_prob_avg` follows train.py:876-941 (checkpoint-outer,
batch-inner; accumulates w * p(target) and scores -log of the mixture). The token-byte table of the reference comes
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


def _reduce_sums(comm, *vals):
    t = torch.stack([v.double() for v in vals])
    if comm is not None:
        comm.all_reduce_sum(t, async_op=False)
    return t.tolist()


@torch.no_grad()
def evaluate_bpb(model, batches, steps, token_bytes, comm=None, num_iterations=None):
    dev = model.get_device()
    total_nats = torch.zeros((), dtype=torch.float64, device=dev)
    total_bytes = torch.zeros((), dtype=torch.float64, device=dev)
    total_loss = torch.zeros((), dtype=torch.float64, device=dev)
    total_tokens = torch.zeros((), dtype=torch.float64, device=dev)
    it = iter(batches)
    for _ in range(steps):
        x, y, _ = next(it)
        loss = model(x, y, loss_reduction="none", num_iterations=num_iterations).view(-1).float()
        y = y.view(-1)
        mask = y != -1
        total_loss += (loss * mask).sum()
        total_tokens += mask.sum()
        nb = token_bytes[y.clamp_min(0)]
        total_nats += (loss * (nb > 0)).sum()
        total_bytes += nb.sum()
    nats, nbytes, loss, ntok = _reduce_sums(comm, total_nats, total_bytes, total_loss, total_tokens)
    bpb = nats / (math.log(2) * nbytes) if nbytes > 0 else float("inf")
    return bpb, (loss / ntok if ntok > 0 else float("inf"))


@torch.no_grad()
def evaluate_prob_avg(model, build_val_loader, ckpt_paths, weights, steps, token_bytes, comm=None, load_fn=None):
    """Mixture-of-checkpoints evaluation: p(y) = sum_c w_c softmax(logits_c)[y]; loss = -log max(p, 1e-40)."""
    from .checkpoint import load_named_params
    dev = model.get_device()
    V = model.config.vocab_size
    loader = build_val_loader()
    xs, ys = [], []
    for _ in range(steps):
        x, y, _ = next(loader)
        xs.append(x.cpu())
        ys.append(y.cpu())
    BT = ys[0].numel()
    acc = torch.zeros(steps, BT, dtype=torch.float32, device=dev)
    for path, w in zip(ckpt_paths, weights):
        ck = torch.load(path, map_location="cpu", weights_only=True)
        (load_fn or load_named_params)(model, ck)
        del ck
        for i, (x, y) in enumerate(zip(xs, ys)):
            yf = y.view(-1).to(dev)
            logits = model(x.to(dev))
            probs = torch.softmax(logits.view(BT, V).float(), dim=-1)
            acc[i].add_(probs[torch.arange(BT, device=dev), yf.clamp_min(0)], alpha=w)
    tn = torch.zeros((), dtype=torch.float64, device=dev)
    tb = torch.zeros((), dtype=torch.float64, device=dev)
    tl = torch.zeros((), dtype=torch.float64, device=dev)
    tt = torch.zeros((), dtype=torch.float64, device=dev)
    for i, y in enumerate(ys):
        yf = y.view(-1).to(dev)
        mask = yf != -1
        lp = acc[i].clamp_min(1e-40).log()
        nb = token_bytes[yf.clamp_min(0)]
        tn += (lp.neg() * (nb > 0)).sum().double()
        tb += nb.sum()
        tl += lp[mask].neg().sum().double()
        tt += mask.sum()
    nats, nbytes, loss, ntok = _reduce_sums(comm, tn, tb, tl, tt)
    bpb = nats / (math.log(2) * nbytes) if nbytes > 0 else float("inf")
    return bpb, (loss / ntok if ntok > 0 else float("inf"))
