"""Batch order of TokenLoader against the reference DataLoader, per rank and across epochs (train.py:765-840)."""
import os

import pytest
import torch

from slowrun_b200.data.loader import TokenLoader
from slowrun_b200.data.synthetic import write_synthetic_corpus
from tests import refload


@pytest.fixture(scope="module")
def corpus(tmp_path_factory):
    d = tmp_path_factory.mktemp("corpus")
    return write_synthetic_corpus(str(d), train_tokens=400_000, val_tokens=60_000)


def test_corpus_format(corpus):
    d = torch.load(corpus[0], weights_only=True)
    assert d["tokens"].dtype == torch.uint16 and d["doc_starts"].dtype == torch.int64
    assert d["bos_id"] == 50256 and d["seq_size"] == 2049
    assert (d["tokens"][d["doc_starts"]].long() == 50256).all()
    assert int(d["tokens"].long().max()) <= 50256


@pytest.mark.parametrize("doc_shuffle", [True, False])
@pytest.mark.parametrize("world,rank", [(1, 0), (2, 1)])
def test_batches_equal_reference(corpus, doc_shuffle, world, rank):
    ref = refload.load_limited()
    if ref is None:
        pytest.skip("reference source not available")
    ref.DataLoader.__init__.__globals__["get_dist_info"] = lambda: (world > 1, rank, rank, world)
    B, T = 2, 256
    r = ref.DataLoader(corpus[0], B, T, device="cpu", doc_shuffle=doc_shuffle)
    m = TokenLoader(corpus[0], B, T, device="cpu", doc_shuffle=doc_shuffle, rank=rank, world_size=world)
    assert r.num_steps == m.num_steps and r.total_tokens == m.total_tokens
    n = 2 * r.num_steps + 3   # crosses two epoch boundaries
    for i in range(n):
        rx, ry, re = next(r)
        mx, my, me = next(m)
        assert re == me, i
        assert torch.equal(rx, mx) and torch.equal(ry, my), i
