"""Step-indexed schedules: learning-rate multiplier with SWA cosine cycles, weight-decay multiplier, Muon momentum
ramp, the tiny track's MTP-weight annealing and recurrence count, the two-hour track's window stages.

Formulas follow the reference scripts (limited: train.py:1083-1111, 1166-1182; tiny: tiny/train.py:221-298,
1291-1326, 1423-1443; two-hour: two_hour/train.py:142-199).
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import numpy as np

from ..config import TrainConfig

MTP_START_WEIGHTS = [1.0, 0.5, 0.25, 0.125]


@dataclass(frozen=True)
class WindowStage:
    start_epoch: int
    end_epoch: int
    short_window: int
    long_window: int


_STAGE_RE = re.compile(r"^\s*(\d+)\s*(?:-\s*(\d+)\s*)?:\s*(\d+)\s*,\s*(\d+)\s*$")


def parse_window_schedule(spec: str, max_seq_len: int) -> Tuple[WindowStage, ...]:
    """Attention-window stages of the two-hour track (two_hour/train.py:143-199). `spec` is a ';'-separated list of
    `first[-last]:short,long` entries, e.g. "1-6:256,768;7-13:768,1792;14-22:1280,2048"; epochs are 1-based and the
    stages must tile the epoch axis from 1 without gaps. Windows are in tokens, short <= long <= max_seq_len."""
    stages = []
    for entry in filter(None, (e.strip() for e in (spec or "").split(";"))):
        m = _STAGE_RE.match(entry)
        if m is None:
            raise ValueError(f"window schedule entry {entry!r} is not of the form first[-last]:short,long")
        first, last, short, long_ = int(m[1]), int(m[2] or m[1]), int(m[3]), int(m[4])
        expected = stages[-1].end_epoch + 1 if stages else 1
        if first != expected or last < first:
            raise ValueError(f"window schedule entry {entry!r}: stages must cover epochs {expected}, {expected + 1}, ... "
                             "in order without gaps")
        if not 0 < short <= long_ <= max_seq_len:
            raise ValueError(f"window schedule entry {entry!r}: need 0 < short <= long <= {max_seq_len}")
        stages.append(WindowStage(first, last, short, long_))
    return tuple(stages)


def window_stage_for_epoch(schedule, epoch) -> Optional[WindowStage]:
    if not schedule:
        return None
    for st in schedule:
        if st.start_epoch <= epoch <= st.end_epoch:
            return st
    if epoch > schedule[-1].end_epoch:
        return schedule[-1]
    raise ValueError(f"No --window-schedule stage covers epoch {epoch}")


class Schedules:
    """All schedules of one run; `num_iterations` is the reference's estimate round(tokens_per_epoch*epochs/batch)."""

    def __init__(self, cfg: TrainConfig, tokens_per_epoch: int):
        self.cfg = cfg
        self.N = round(tokens_per_epoch * cfg.num_epochs / cfg.total_batch_size)
        self.steps_per_epoch = self.N / cfg.num_epochs
        self.swa_start = (self.N - cfg.swa_last_epochs * self.steps_per_epoch) if cfg.swa_last_epochs > 0 else -1
        self.tiny = cfg.track == "tiny"
        if self.tiny:
            self.wd_s1 = round(cfg.wd_phase1_epoch / cfg.num_epochs * self.N)
            self.wd_s2 = round(cfg.wd_phase2_epoch / cfg.num_epochs * self.N)

    # learning rate -------------------------------------------------------------------------------
    def base_lr_multiplier(self, it: int) -> float:
        c, N = self.cfg, self.N
        warmup = round(c.warmup_ratio * N)
        warmdown = round(c.warmdown_ratio * N)
        if warmup > 0 and it < warmup:
            return (it + 1) / warmup
        if warmdown <= 0 or it <= N - warmdown:
            return 1.0
        progress = (N - it) / warmdown
        shaped = progress ** c.warmdown_power
        return shaped + (1 - shaped) * c.final_lr_frac

    def lr_multiplier(self, it: int) -> float:
        lrm = self.base_lr_multiplier(it)
        if self.swa_start >= 0 and it >= self.swa_start:
            cyc = (it - self.swa_start) % self.steps_per_epoch
            base = max(lrm, 0.05)
            lrm = 0.05 + (base - 0.05) * (1 + math.cos(math.pi * cyc / self.steps_per_epoch)) / 2
        return lrm

    # weight decay --------------------------------------------------------------------------------
    def wd_multiplier(self, it: int) -> float:
        c = self.cfg
        if self.tiny:
            wd = float(np.interp(it, [0, self.wd_s1, self.wd_s2, self.N], [c.weight_decay, c.weight_decay, c.wd_mid, c.wd_end]))
            return wd / c.weight_decay if c.weight_decay > 0 else 0.0
        if self.swa_start >= 0 and it >= self.swa_start:
            frac = ((it - self.swa_start) % self.steps_per_epoch) / self.steps_per_epoch
            return c.wd_swa_low + (c.wd_swa_high - c.wd_swa_low) * frac
        t = it / self.N
        if t < c.wd_pre_hold_frac:
            return 1.0
        swa_frac = self.swa_start / self.N if self.swa_start > 0 else 1.0
        d = (t - c.wd_pre_hold_frac) / max(swa_frac - c.wd_pre_hold_frac, 1e-6)
        d = min(max(d, 0.0), 1.0)
        return 1.0 - (1.0 - c.wd_swa_low) * d

    @staticmethod
    def muon_momentum(it: int) -> float:
        f = min(it / 300, 1)
        return (1 - f) * 0.85 + f * 0.95

    def apply(self, param_groups, it: int):
        """Write lr / weight_decay / momentum of step `it` into the optimizer's groups (train.py:1176-1182)."""
        lrm, wdm = self.lr_multiplier(it), self.wd_multiplier(it)
        for g in param_groups:
            g["lr"] = g["initial_lr"] * lrm
            g["weight_decay"] = g["initial_wd"] * wdm
            if g["kind"] == "muon":
                g["momentum"] = self.muon_momentum(it)
        return lrm, wdm

    # tiny: MTP weights and recurrence ---------------------------------------------------------------
    def mtp_weights(self, it: int):
        c = self.cfg
        n = max(1, min(c.mtp_predict, len(MTP_START_WEIGHTS)))
        w = [1.0]
        if n > 1:
            f = min(1.0, it / max(1, self.N))
            A = c.mtp_anneal_frac
            for k in range(1, n):
                s0 = (n - 1 - k) / (n - 1) * A
                s1 = (n - k) / (n - 1) * A
                if f <= s0:
                    frac = 1.0
                elif f >= s1:
                    frac = 0.0
                else:
                    frac = 1.0 - (f - s0) / (s1 - s0)
                w.append(MTP_START_WEIGHTS[k] * frac)
        return w

    def recurrence_stages(self):
        c = self.cfg
        mx, mn = c.model.num_iterations, c.min_iterations
        if c.iteration_schedule == "constant":
            return ((0.0, 1.0, mx),)
        t = min(max(c.iteration_transition_ratio, 0.0), 1.0)
        if mn == mx or t >= 1.0 - 1e-9:
            return ((0.0, 1.0, mx),)
        if t <= 1e-9:
            return ((0.0, 1.0, mn),)
        return ((0.0, 1.0 - t, mn), (1.0 - t, 1.0, mx))

    def num_recurrences(self, it: int) -> int:
        stages = self.recurrence_stages()
        if self.N <= 0:
            return stages[-1][2]
        frac = min(max(it / self.N, 0.0), 1.0)
        for i, (a, b, k) in enumerate(stages):
            if frac < b or i == len(stages) - 1:
                return k
        return stages[-1][2]
