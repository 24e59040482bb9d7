"""Synthetic Zipf-distributed corpus in the reference's on-disk format.

The file is the dict that prepare_data.py writes (prepare_data.py:55-62): uint16 `tokens`, int64 `doc_starts`
(every document starts with the BOS id 50256), `bos_id`, `seq_shuffle_seed`, `seq_size`. Token ids are i.i.d.
Zipf(s) over the 50257-entry GPT-2 vocabulary (BOS only appears as the document delimiter); document lengths are
geometric with a configurable mean. Used by the benchmarks and tests, where no dataset can be downloaded.
"""
from __future__ import annotations

import os

import numpy as np
import torch

BOS_ID = 50256
SEQ_SIZE = 2049


def zipf_tokens(n: int, vocab: int = 50256, s: float = 1.1, seed: int = 0) -> np.ndarray:
    """n ids in [0, vocab) with P(rank k) ~ 1/(k+1)^s, ranks mapped to ids by a fixed permutation."""
    rng = np.random.default_rng(seed)
    w = 1.0 / np.power(np.arange(1, vocab + 1, dtype=np.float64), s)
    cdf = np.cumsum(w / w.sum())
    ranks = np.searchsorted(cdf, rng.random(n), side="right").clip(max=vocab - 1)
    perm = np.random.default_rng(12345).permutation(vocab)
    return perm[ranks].astype(np.uint16)


def make_corpus(num_tokens: int, mean_doc_len: int = 700, s: float = 1.1, seed: int = 0):
    rng = np.random.default_rng(seed + 1)
    tokens = zipf_tokens(num_tokens, s=s, seed=seed)
    starts = [0]
    pos = 0
    while True:
        pos += int(rng.geometric(1.0 / mean_doc_len)) + 1
        if pos >= num_tokens:
            break
        starts.append(pos)
    doc_starts = np.asarray(starts, dtype=np.int64)
    tokens[doc_starts] = BOS_ID
    return tokens, doc_starts


def write_datafile(path: str, tokens: np.ndarray, doc_starts: np.ndarray, shuffle_seed: int):
    assert doc_starts[0] == 0 and np.all(tokens[doc_starts] == BOS_ID)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    torch.save({
        "tokens": torch.from_numpy(tokens.copy()),
        "doc_starts": torch.from_numpy(doc_starts.copy()),
        "bos_id": int(BOS_ID),
        "seq_shuffle_seed": int(shuffle_seed),
        "seq_size": int(SEQ_SIZE),
    }, path)


def write_synthetic_corpus(out_dir: str, train_tokens: int = 100_000_000, val_tokens: int = 10_000_000,
                           s: float = 1.1, seed: int = 0):
    """Writes fineweb_train.pt / fineweb_val.pt under out_dir (same names the entry points default to)."""
    tr = os.path.join(out_dir, "fineweb_train.pt")
    va = os.path.join(out_dir, "fineweb_val.pt")
    t, d = make_corpus(val_tokens, s=s, seed=seed + 100)
    write_datafile(va, t, d, 42)
    t, d = make_corpus(train_tokens, s=s, seed=seed)
    write_datafile(tr, t, d, 43)
    return tr, va
