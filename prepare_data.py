"""Builds fineweb_data/fineweb_{train,val}.pt.

    python prepare_data.py                       # FineWeb sample-10BT through `datasets` + `tiktoken` (needs network)
    python prepare_data.py --synthetic           # Zipf(1.1) tokens, no network: the corpus the benchmarks use
    python prepare_data.py --train_tokens 100_000_000 --val_tokens 10_000_000 --local_dir fineweb_data

Output format, split order (validation tokens first, then training), per-document BOS and the SHA-256 check of the
real corpus follow the reference's prepare_data.py (prepare_data.py:25-134): a dict with uint16 `tokens`, int64
`doc_starts`, `bos_id` 50256, `seq_shuffle_seed` (42 validation / 43 training) and `seq_size` 2049.
"""
import argparse
import hashlib
import os

import numpy as np

from slowrun_b200.data.synthetic import BOS_ID, write_datafile, write_synthetic_corpus

VAL_SHUFFLE_SEED, TRAIN_SHUFFLE_SEED = 42, 43
EXPECTED_SHA256 = {
    "fineweb_val.pt": "6868ed375b289a89c72c2f9df1ecbdcff700c4b9478ca806435d2dbfad8573b1",
    "fineweb_train.pt": "36e7c95c1e7f6ed952fb002d76a03044e8617fea7e696a68d7dc1ce78465dcaf",
}


def sha256_of(path):
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def take_tokens(doc_iter, encoder, budget):
    """Consume documents until `budget` tokens are collected; every document is prefixed with BOS."""
    out = np.empty(budget, dtype=np.uint16)
    starts, n = [], 0
    for doc in doc_iter:
        ids = [BOS_ID] + encoder.encode_ordinary(doc["text"])
        starts.append(n)
        k = min(len(ids), budget - n)
        out[n:n + k] = ids[:k]
        n += k
        if n >= budget:
            break
    return out[:n], np.asarray(starts, dtype=np.int64)


def build_from_fineweb(train_tokens, val_tokens, local_dir):
    try:
        import tiktoken
        from datasets import load_dataset
        enc = tiktoken.get_encoding("gpt2")
        stream = iter(load_dataset("HuggingFaceFW/fineweb", name="sample-10BT", split="train", streaming=True))
    except Exception as e:  # noqa: BLE001
        raise SystemExit(f"FineWeb / GPT-2 vocabulary not reachable ({type(e).__name__}: {e}).\n"
                         "Use --synthetic for an offline corpus in the same format.")
    assert enc._special_tokens["<|endoftext|>"] == BOS_ID
    os.makedirs(local_dir, exist_ok=True)
    val, val_starts = take_tokens(stream, enc, val_tokens)
    trn, trn_starts = take_tokens(stream, enc, train_tokens)
    paths = (os.path.join(local_dir, "fineweb_val.pt"), os.path.join(local_dir, "fineweb_train.pt"))
    write_datafile(paths[0], val, val_starts, VAL_SHUFFLE_SEED)
    write_datafile(paths[1], trn, trn_starts, TRAIN_SHUFFLE_SEED)
    for p in paths:
        digest, want = sha256_of(p), EXPECTED_SHA256.get(os.path.basename(p))
        default_sizes = train_tokens == 100_000_000 and val_tokens == 10_000_000
        if want and default_sizes:
            assert digest == want, f"hash mismatch for {p}: {digest} != {want}"
        print(f"{p}: sha256 {digest}")


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description="Prepare the Slowrun token files")
    ap.add_argument("--train_tokens", type=int, default=100_000_000)
    ap.add_argument("--val_tokens", type=int, default=10_000_000)
    ap.add_argument("--local_dir", type=str, default="fineweb_data")
    ap.add_argument("--synthetic", action="store_true", help="write a Zipf(s=1.1) corpus instead of FineWeb")
    ap.add_argument("--zipf-s", type=float, default=1.1)
    a = ap.parse_args()
    if a.synthetic:
        print(write_synthetic_corpus(a.local_dir, a.train_tokens, a.val_tokens, s=a.zipf_s))
    else:
        build_from_fineweb(a.train_tokens, a.val_tokens, a.local_dir)
