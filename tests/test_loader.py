"""Batch order of TokenLoader against the reference DataLoader, per rank and across epochs (train.py:765-840)."""
import os

import pytest
import torch

from slowrun_b200.data.loader import EnsembleTokenLoader, TokenLoader
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


@pytest.mark.parametrize("world,rank", [(1, 0), (2, 1)])
def test_ensemble_loader_equals_reference_unlimited_loader(corpus, world, rank):
    ref = refload.load_unlimited_loaders()
    if ref is None:
        pytest.skip("reference source not available")
    B, T, seed, fit = 2, 256, 3, 20_000
    docs, dseed = ref._load_new_format_file(corpus[0])
    fit_docs, train_docs, _ = ref._carve_fitness_docs(docs, fit)
    r = ref.DataLoader(None, B, T, device="cpu", seed=seed, dp_rank=rank, dp_world_size=world, doc_shuffle=True,
                       doc_tokens=train_docs, default_shuffle_seed=dseed)
    m = EnsembleTokenLoader(corpus[0], B, T, device="cpu", seed=seed, rank=rank, world_size=world, fitness_tokens=fit)
    assert r.num_steps == m.num_steps and r.total_tokens == m.total_tokens
    for i in range(2 * r.num_steps + 3):
        rx, ry, re = next(r)
        mx, my, me = next(m)
        assert re == me, i
        assert torch.equal(rx, mx) and torch.equal(ry, my), i
    # the held-out slice, read the way the reference's p(ground truth) cache reads it
    fseqs = ref._build_seqs_from_docs(fit_docs, T + 1)
    rv = ref.DDPValLoader(None, 4, T, rank=rank, world_size=world, device="cpu", seed=0, seqs=fseqs)
    mv = EnsembleTokenLoader(corpus[0], 4, T, device="cpu", seed=0, rank=rank, world_size=world, fitness_tokens=fit,
                             fitness_only=True)
    assert rv.num_steps == mv.num_steps
    for i in range(rv.num_steps):
        rx, ry, _ = next(rv)
        mx, my, _ = next(mv)
        assert torch.equal(rx, mx) and torch.equal(ry, my), i


def test_loader_state_round_trip(corpus):
    a = TokenLoader(corpus[0], 2, 256, device="cpu", doc_shuffle=True)
    for _ in range(a.num_steps + 5):
        next(a)
    st = a.state()
    b = TokenLoader(corpus[0], 2, 256, device="cpu", doc_shuffle=True)
    b.restore(st)
    for _ in range(a.num_steps):
        xa, ya, ea = next(a)
        xb, yb, eb = next(b)
        assert ea == eb and torch.equal(xa, xb) and torch.equal(ya, yb)


def test_legacy_chunked_dataset(tmp_path):
    """research/hybrid_attn/train.py:1146-1186, 1208-1216, 1246-1250: rows of the pre-chunked file in file order, dealt
    [step, rank, B]; later epochs only permute the order of a rank's steps (seed = epoch)."""
    import torch
    from slowrun_b200.data.loader import TokenLoader
    B_file, S = 6, 9
    g = torch.Generator().manual_seed(0)
    chunks = [torch.randint(0, 1000, (B_file * S,), generator=g, dtype=torch.int32) for _ in range(4)]
    valid = [6, 6, 4, 6]
    path = str(tmp_path / "legacy.pt")
    torch.save({"chunks": chunks, "valid_counts": valid, "batch_size": B_file, "sequence_size": S}, path)
    rows = torch.cat([c.view(B_file, S)[:v] for c, v in zip(chunks, valid)], 0).long()      # 22 rows
    for rank in (0, 1):
        ld = TokenLoader(path, 2, S - 1, device="cpu", doc_shuffle=True, rank=rank, world_size=2)
        assert ld.doc_shuffle is False and ld.num_steps == 5 and ld.total_tokens == 20 * (S - 1)
        mine = rows[:20].view(5, 2, 2, S)[:, rank]
        for s_ in range(5):
            x, y, ep = next(ld)
            assert ep == 1 and torch.equal(x, mine[s_][:, :-1]) and torch.equal(y, mine[s_][:, 1:])
        perm = torch.randperm(5, generator=torch.Generator().manual_seed(2))
        for s_ in range(5):
            x, y, ep = next(ld)
            assert ep == 2 and torch.equal(x, mine[perm[s_]][:, :-1])
    with pytest.raises(ValueError, match="not a recognized dataset format"):
        torch.save({"foo": torch.zeros(3)}, str(tmp_path / "bad.pt"))
        TokenLoader(str(tmp_path / "bad.pt"), 2, 8, device="cpu")
