"""Epoch-shuffling token loader.

The batch order, per rank and per epoch, is bit-for-bit the one the reference's `DataLoader` yields
(train.py:765-840; unlimited variant unlimited/train.py:765-964): that order is part of the training recipe.
How it is produced is different. The corpus stays ONE int32 token tensor plus a table of document offsets; an
epoch is described by a document order (an index vector that the per-epoch permutations act on) and a sequence
permutation, and a rank materialises only ITS rows of the epoch: for every sequence it owns, the positions of the
virtual concatenated stream are mapped back to corpus positions with one `searchsorted` over the cumulative document
lengths and fetched with one gather. Nothing is concatenated, no per-document tensors exist, and a rank touches
1/world of the tokens per epoch. The per-rank table lives in pinned host memory as int32; each batch is one
asynchronous H2D copy on a side stream, issued one step ahead and widened to int64 on the device.
"""
from __future__ import annotations

import os

import numpy as np
import torch

from ..config import BOS_ID


class Corpus:
    """Tokens of a `.pt` corpus file (prepare_data.py format) and its document table."""

    CHUNKED_KEYS = {"chunks", "valid_counts", "batch_size", "sequence_size"}
    FLAT_KEYS = {"tokens", "doc_starts", "bos_id", "seq_shuffle_seed"}

    def __init__(self, filepath):
        data = torch.load(filepath, weights_only=True)
        self.fixed_rows = None
        if self.CHUNKED_KEYS.issubset(data):
            # Legacy pre-chunked files (research/hybrid_attn/train.py:1146-1186): a list of [batch_size, sequence_size]
            # chunks of which the first valid_counts[i] rows count. The windows are fixed, so there is no document
            # table and nothing to shuffle but the order of a rank's steps.
            B, S = int(data["batch_size"]), int(data["sequence_size"])
            rows = [c.view(B, S)[:int(v)] for c, v in zip(data["chunks"], data["valid_counts"])]
            self.fixed_rows = torch.cat(rows, 0).to(torch.int32)
            self.tokens = self.fixed_rows.reshape(-1)
            self.starts = torch.zeros(1, dtype=torch.int64)
            self.lens = torch.tensor([self.tokens.numel()], dtype=torch.int64)
            self.seq_shuffle_seed = 0
            return
        if not self.FLAT_KEYS.issubset(data):
            raise ValueError(f"{filepath} is not a recognized dataset format. Expected flat keys {sorted(self.FLAT_KEYS)} or "
                             f"chunked keys {sorted(self.CHUNKED_KEYS)}, found [{', '.join(sorted(data.keys()))}].")
        bos_id = int(data["bos_id"])
        if bos_id != BOS_ID:
            raise ValueError(f"corpus was tokenised with bos_id {bos_id}, this loader expects {BOS_ID}")
        self.tokens = data["tokens"].to(torch.int32)
        self.starts = data["doc_starts"].to(torch.int64)
        ends = torch.cat([self.starts[1:], torch.tensor([self.tokens.numel()], dtype=torch.int64)])
        self.lens = ends - self.starts
        self.seq_shuffle_seed = data["seq_shuffle_seed"]

    @property
    def num_docs(self):
        return self.starts.numel()


class EpochStream:
    """The virtual token stream "documents `order[0]`, `order[1]`, ... back to back" of one epoch."""

    def __init__(self, corpus: Corpus, order: torch.Tensor):
        self.corpus = corpus
        lens = corpus.lens[order]
        self.first = torch.cumsum(lens, 0) - lens                 # stream position where each document begins
        self.src0 = corpus.starts[order]                          # corpus position where it begins
        self.length = int(lens.sum())

    def rows(self, seq_ids: torch.Tensor, seq_size: int) -> torch.Tensor:
        """int32 [len(seq_ids), seq_size]: windows `seq_ids[i] * seq_size ...` of the stream, fetched from the corpus."""
        pos = (seq_ids.to(torch.int64) * seq_size).unsqueeze(1) + torch.arange(seq_size, dtype=torch.int64)
        doc = torch.searchsorted(self.first, pos.reshape(-1), right=True) - 1
        src = self.src0[doc] + (pos.reshape(-1) - self.first[doc])
        return self.corpus.tokens[src].view(len(seq_ids), seq_size)


def _generator(seed: int) -> torch.Generator:
    g = torch.Generator()
    g.manual_seed(int(seed))
    return g


class TokenLoader:
    """Infinite iterator of (x [B, T], y [B, T], epoch) for the limited, tiny and two-hour tracks.

    doc_shuffle on: before every epoch after the first the document order is permuted again (seed = epoch, acting on
    the previous order), the stream is cut into windows of T + 1 tokens, the windows are permuted (seed = epoch +
    1000), the tail that does not fill a step of B * world windows is dropped and step s of rank r is windows
    [s, r, :] of the [steps, world, B] arrangement. doc_shuffle off: file order, one fixed window permutation from
    the seed stored in the file, and per epoch only the order of this rank's steps is re-permuted (seed = epoch)."""

    def __init__(self, filepath, B, T, device="cuda", doc_shuffle=False, rank=0, world_size=1, prefetch=True):
        self.corpus = Corpus(filepath)
        self.rank, self.world_size = rank, world_size
        self.device = torch.device(device)
        self.B, self.T, self.seq_size = B, T, T + 1
        self.doc_shuffle = doc_shuffle
        if self.corpus.fixed_rows is not None:
            if self.corpus.fixed_rows.size(1) != self.seq_size:
                raise ValueError(f"Data sequence_size {self.corpus.fixed_rows.size(1)} != T+1={T + 1}")
            if doc_shuffle and int(os.environ.get("RANK", 0)) == 0:
                print(f"Warning: {filepath} is a legacy chunked dataset; document shuffling is unavailable until the data "
                      "is regenerated with prepare_data.py.")
            self.doc_shuffle = False
        self.epoch = 1
        self.order = torch.arange(self.corpus.num_docs)
        self._cuda = self.device.type == "cuda"
        self._stream = torch.cuda.Stream(device=self.device) if (self._cuda and prefetch) else None
        self._next = None
        self.h2d_bytes_per_batch = B * self.seq_size * 4
        self._plan_epoch()

    # ------------------------------------------------------------------ what this rank reads in the current epoch
    def _window_permutation(self, num_seqs):
        if self.corpus.fixed_rows is not None:
            return torch.arange(num_seqs)                   # legacy chunked files: rows are used in file order
        if self.doc_shuffle:
            return torch.randperm(num_seqs, generator=_generator(self.epoch + 1000))
        return torch.from_numpy(np.random.RandomState(self.corpus.seq_shuffle_seed).permutation(num_seqs))

    def _rank_share(self, perm):
        """(window ids of this rank in step order, steps, windows used by all ranks)"""
        per_step = self.B * self.world_size
        steps = perm.numel() // per_step
        mine = perm[:steps * per_step].view(steps, self.world_size, self.B)[:, self.rank]
        return mine.reshape(-1), steps, steps * per_step

    def _plan_epoch(self):
        stream = EpochStream(self.corpus, self.order)
        ids, steps, used = self._rank_share(self._window_permutation(stream.length // self.seq_size))
        self._set_table(stream.rows(ids, self.seq_size).view(steps, self.B, self.seq_size))
        self.num_steps = steps
        self.total_tokens = used * self.T
        self.pos = 0

    def _set_table(self, t):
        t = t.contiguous()
        self.rank_data = t.pin_memory() if self._cuda else t
        self._next = None

    def _advance_epoch(self):
        self.epoch += 1
        if int(os.environ.get("RANK", 0)) == 0:
            print(f"Starting epoch {self.epoch}")
        if self.doc_shuffle:
            self.order = self.order[torch.randperm(self.order.numel(), generator=_generator(self.epoch))]
            self._plan_epoch()
        else:
            self._set_table(self.rank_data[torch.randperm(self.num_steps, generator=_generator(self.epoch))])
            self.pos = 0

    # ------------------------------------------------------------------ transport
    def __iter__(self):
        return self

    def _issue(self):
        """Start the copy of the batch at self.pos (rolling the epoch if needed)."""
        if self.pos >= self.num_steps:
            self._advance_epoch()
        host = self.rank_data[self.pos]
        self.pos += 1
        if self._stream is not None:
            with torch.cuda.stream(self._stream):
                dev = host.to(self.device, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self._stream)
            return dev, ev, self.epoch
        return host.to(self.device, non_blocking=True), None, self.epoch

    def __next__(self):
        if self._next is None:
            self._next = self._issue()
        dev, ev, epoch = self._next
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
            dev.record_stream(torch.cuda.current_stream())
        batch = dev.long()
        x, y = batch[:, :-1].contiguous(), batch[:, 1:].contiguous()
        # The next copy is issued now unless it would roll the epoch: the epoch reported with a batch is the loader's
        # epoch at the moment that batch was taken.
        self._next = None
        if self._stream is not None and self.pos < self.num_steps:
            self._next = self._issue()
        return x, y, epoch

    # ------------------------------------------------------------------ resume support
    def state(self, rewind: int = 0) -> dict:
        """Position of the next batch the CONSUMER will see (a prefetched but unconsumed batch is counted as unread).
        `rewind=1`: the consumer still holds the batch it was given last and wants it delivered again after a restore
        (a trainer that fetches one batch ahead). The epoch never rolls between a batch and the call that follows it,
        so the rewound position lies in the current epoch."""
        pos = self.pos - (1 if self._next is not None else 0) - int(rewind)
        if pos < 0:
            raise ValueError("cannot rewind past the start of the epoch")
        return {"epoch": self.epoch, "pos": pos, "order": self.order.clone()}

    def restore(self, st: dict):
        """Re-create the table of the saved epoch and continue at the saved step. With doc_shuffle off the cumulative
        step permutations of the elapsed epochs are replayed."""
        target_epoch, pos = int(st["epoch"]), int(st["pos"])
        self._next = None
        if self.doc_shuffle:
            self.epoch = target_epoch
            self.order = st["order"].clone()
            self._plan_epoch()
        else:
            self.epoch = 1
            self._plan_epoch()
            while self.epoch < target_epoch:
                self.epoch += 1
                self._set_table(self.rank_data[torch.randperm(self.num_steps, generator=_generator(self.epoch))])
        self.pos = pos


class EnsembleTokenLoader(TokenLoader):
    """Loader of the unlimited track (unlimited/train.py:765-964): a per-model seed, steps dealt round-robin to the
    data-parallel ranks, and a held-out "fitness" slice taken from the front of the file at document granularity.
    Epoch e of the model with seed s: the document order is permuted again with seed s * 1009 + e + 1000 (also
    before the first epoch), windows with seed s * 1009 + e + 2000, the step list is cut to a multiple of the
    data-parallel size and rank r takes steps r, r + world, ... With `fitness_only` the loader serves the held-out
    documents instead, the way the reference's p(ground truth) cache reads them (unlimited/train.py:1002-1009): windows
    of the held-out stream permuted with seed `seed + epoch`, step s of rank r = windows [s, r, :]."""

    def __init__(self, filepath, B, T, device="cuda", seed=0, rank=0, world_size=1, fitness_tokens=0,
                 fitness_only=False, prefetch=True):
        self.seed = int(seed)
        self.fitness_tokens = int(fitness_tokens)
        self.fitness_only = fitness_only
        self.fitness_order = None
        self._keep_order = False
        super().__init__(filepath, B, T, device=device, doc_shuffle=True, rank=rank, world_size=world_size,
                         prefetch=prefetch)

    def _carve(self):
        """Split the document list once: the shortest prefix holding at least `fitness_tokens` tokens is held out."""
        if self.fitness_order is not None:
            return
        n = self.corpus.num_docs
        cut = 0
        if self.fitness_tokens > 0:
            csum = torch.cumsum(self.corpus.lens, 0)
            cut = min(int(torch.searchsorted(csum, self.fitness_tokens, right=False)) + 1, n)
        self.fitness_order = torch.arange(cut)
        self.order = torch.arange(cut, n)

    def _plan_epoch(self):
        self._carve()
        if self.fitness_only:
            stream = EpochStream(self.corpus, self.fitness_order)
            perm = torch.randperm(stream.length // self.seq_size, generator=_generator(self.seed + self.epoch))
            ids, steps, used = self._rank_share(perm)
            self._set_table(stream.rows(ids, self.seq_size).view(steps, self.B, self.seq_size))
            self.num_steps, self.total_tokens, self.pos = steps, used * self.T, 0
            return
        else:
            base = self.seed * 1009 + self.epoch
            if not self._keep_order:
                self.order = self.order[torch.randperm(self.order.numel(), generator=_generator(base + 1000))]
            stream = EpochStream(self.corpus, self.order)
            perm = torch.randperm(stream.length // self.seq_size, generator=_generator(base + 2000))
        steps_total = (perm.numel() // self.B // self.world_size) * self.world_size
        used = steps_total * self.B
        mine = perm[:used].view(steps_total, self.B)[self.rank::self.world_size]
        steps = steps_total // self.world_size
        self._set_table(stream.rows(mine.reshape(-1), self.seq_size).view(steps, self.B, self.seq_size))
        self.num_steps = steps
        self.total_tokens = used * self.T
        self.pos = 0

    def _advance_epoch(self):
        self.epoch += 1
        self._plan_epoch()

    def restore(self, st: dict):
        """`st["order"]` is the document order of the saved epoch (already permuted for it)."""
        self._carve()
        self.epoch, self.order = int(st["epoch"]), st["order"].clone()
        self._keep_order = True
        try:
            self._plan_epoch()
        finally:
            self._keep_order = False
        self.pos = int(st["pos"])
