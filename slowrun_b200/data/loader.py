"""Epoch-shuffling token loader with the reference's exact ordering.

Order of batches, per rank and per epoch, is the one `DataLoader` of the reference produces (train.py:765-840):
documents are cumulatively re-permuted each epoch with seed = epoch, concatenated, cut into T+1 windows, the
windows permuted with seed = epoch + 1000, the tail dropped, and step s of rank r is rows
[s, r, :, :] of the [steps, world, B, T+1] view. With doc_shuffle off the stored numpy permutation is applied once
and only the step order is reshuffled per epoch.

What differs is the transport: the per-rank table is kept as int32 in pinned host memory and each batch is a
single asynchronous H2D copy on a side stream, prefetched one step ahead, widened to int64 on the device.
"""
from __future__ import annotations

import os

import numpy as np
import torch

from ..config import BOS_ID


class TokenLoader:
    def __init__(self, filepath, B, T, device="cuda", doc_shuffle=False, rank=0, world_size=1, prefetch=True,
                 seed_fn=None):
        data = torch.load(filepath, weights_only=True)
        all_tokens = data["tokens"].long()
        raw_doc_starts = data["doc_starts"].long()
        bos_id = int(data["bos_id"])
        assert bos_id == BOS_ID, f"data bos_id {bos_id} != expected {BOS_ID}"
        doc_ends = torch.cat([raw_doc_starts[1:], torch.tensor([all_tokens.numel()])])
        self.doc_tokens = [all_tokens[s:e] for s, e in zip(raw_doc_starts.tolist(), doc_ends.tolist())]
        self.default_shuffle_seed = data["seq_shuffle_seed"]
        self.rank, self.world_size = rank, world_size
        self.device = torch.device(device)
        self.B, self.T, self.seq_size = B, T, T + 1
        self.doc_shuffle = doc_shuffle
        self.epoch = 1
        self._cuda = self.device.type == "cuda"
        self._stream = torch.cuda.Stream(device=self.device) if (self._cuda and prefetch) else None
        self._next = None
        self.h2d_bytes_per_batch = B * self.seq_size * 4
        self._build_batches()

    def _build_batches(self):
        tokens = torch.cat(self.doc_tokens)
        num_seqs = len(tokens) // self.seq_size
        all_seqs = tokens[:num_seqs * self.seq_size].view(num_seqs, self.seq_size)
        if self.doc_shuffle:
            g = torch.Generator()
            g.manual_seed(self.epoch + 1000)
            all_seqs = all_seqs[torch.randperm(num_seqs, generator=g)]
        else:
            perm = np.random.RandomState(self.default_shuffle_seed).permutation(num_seqs)
            all_seqs = all_seqs[torch.from_numpy(perm)]
        seqs_per_step = self.B * self.world_size
        num_steps = len(all_seqs) // seqs_per_step
        usable = num_steps * seqs_per_step
        all_seqs = all_seqs[:usable].view(num_steps, self.world_size, self.B, self.seq_size)
        self._set_rank_data(all_seqs[:, self.rank])
        self.num_steps = num_steps
        self.total_tokens = usable * self.T
        self.pos = 0

    def _set_rank_data(self, t):
        t = t.to(torch.int32).contiguous()
        self.rank_data = t.pin_memory() if self._cuda else t
        self._next = None

    def __iter__(self):
        return self

    def _next_epoch(self):
        self.epoch += 1
        if int(os.environ.get("RANK", 0)) == 0:
            print(f"Starting epoch {self.epoch}")
        if self.doc_shuffle:
            g = torch.Generator()
            g.manual_seed(self.epoch)
            perm = torch.randperm(len(self.doc_tokens), generator=g)
            self.doc_tokens = [self.doc_tokens[i] for i in perm.tolist()]
            self._build_batches()
        else:
            self.pos = 0
            g = torch.Generator()
            g.manual_seed(self.epoch)
            self._set_rank_data(self.rank_data[torch.randperm(self.num_steps, generator=g)])

    def _issue(self):
        """Start the copy of the batch at self.pos (rolling the epoch if needed); returns (device int32, epoch)."""
        if self.pos >= self.num_steps:
            self._next_epoch()
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
        # prefetch the following batch while this one is consumed (does not roll the visible epoch early:
        # the epoch returned with a batch is the loader's epoch after that batch was taken, as in the reference)
        x, y = batch[:, :-1].contiguous(), batch[:, 1:].contiguous()
        self._next = None
        if self._stream is not None and self.pos < self.num_steps:
            self._next = self._issue()
        return x, y, epoch


class EnsembleTokenLoader(TokenLoader):
    """Loader of the unlimited track: per-model seed, step interleaving over data-parallel ranks, and a held-out
    "fitness" slice carved from the front of the training file at document granularity
    (unlimited/train.py:765-964). Ordering per epoch e of a model with seed s: documents permuted (cumulatively)
    with seed s*1009 + e + 1000, windows permuted with seed s*1009 + e + 2000, the step list truncated to a multiple
    of the data-parallel size and rank r takes steps r, r + world, ...
    """

    def __init__(self, filepath, B, T, device="cuda", seed=0, rank=0, world_size=1, fitness_tokens=0,
                 fitness_only=False, prefetch=True):
        self.seed = int(seed)
        self.fitness_tokens = int(fitness_tokens)
        self.fitness_only = fitness_only
        self._carved = False
        super().__init__(filepath, B, T, device=device, doc_shuffle=True, rank=rank, world_size=world_size,
                         prefetch=prefetch)

    def _carve(self):
        if self._carved:
            return
        self._carved = True
        if self.fitness_tokens <= 0:
            self.fitness_docs = []
            return
        n, cut = 0, 0
        for cut, d in enumerate(self.doc_tokens):
            if n >= self.fitness_tokens:
                break
            n += len(d)
        else:
            cut = len(self.doc_tokens)
        self.fitness_docs = self.doc_tokens[:cut]
        self.doc_tokens = self.doc_tokens[cut:]

    def _build_batches(self):
        self._carve()
        if self.fitness_only:
            tokens = torch.cat(self.fitness_docs) if self.fitness_docs else torch.zeros(0, dtype=torch.long)
            num_seqs = len(tokens) // self.seq_size
            all_seqs = tokens[:num_seqs * self.seq_size].view(num_seqs, self.seq_size)
        else:
            g = torch.Generator()
            g.manual_seed(self.seed * 1009 + self.epoch + 1000)
            perm = torch.randperm(len(self.doc_tokens), generator=g)
            self.doc_tokens = [self.doc_tokens[i] for i in perm.tolist()]
            tokens = torch.cat(self.doc_tokens)
            num_seqs = len(tokens) // self.seq_size
            all_seqs = tokens[:num_seqs * self.seq_size].view(num_seqs, self.seq_size)
            g.manual_seed(self.seed * 1009 + self.epoch + 2000)
            all_seqs = all_seqs[torch.randperm(num_seqs, generator=g)]
        steps_total = len(all_seqs) // self.B
        steps_total = (steps_total // self.world_size) * self.world_size
        usable = steps_total * self.B
        all_seqs = all_seqs[:usable].view(steps_total, self.B, self.seq_size)
        self._set_rank_data(all_seqs[self.rank::self.world_size])
        self.num_steps = steps_total // self.world_size
        self.total_tokens = usable * self.T
        self.pos = 0

    def _next_epoch(self):
        self.epoch += 1
        self._build_batches()
