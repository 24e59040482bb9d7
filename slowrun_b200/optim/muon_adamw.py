"""Sharded Muon + AdamW (optimizer state and update work split over data-parallel ranks).

Update rule and hyper-parameter plumbing follow the reference's DistMuonAdamW (train.py:594-760): Nesterov momentum,
MuonEq-R row normalisation, five "Polar Express" Newton-Schulz iterations in bf16, NorMuon variance reduction and
cautious weight decay for matrices; AdamW (decay first, bias-corrected) for embeddings, head and scalars.

What is organised differently:
  * gradients, parameters and bf16 shadows live in stacked arenas (`arena.py`), so reduce-scatter inputs and the
    owned stacks are slices, never copies;
  * the Newton-Schulz products run on the tcgen05 GEMM with symmetric-output tiles (X X^T and bA + cA^2 only compute
    the upper triangle) and the polynomial/axpy terms fused into the GEMM epilogue;
  * what is all-gathered is the bf16 orthogonalised update, applied by every rank to its own replica
    (`P -= lr*U + lr*wd*P*[U*P >= 0]`), instead of the updated fp32 parameters: half the bytes, and no padding
    traffic for one-matrix groups beyond the zero chunk;
  * all small parameters share one gradient buffer and one all-reduce.
"""
from __future__ import annotations

import os
from typing import List

import torch

from ..ops import _lib
from ..ops.gemm import gemm
from .arena import ParamArena, SMALL_NUMEL

# Polar Express coefficients (train.py:586-592)
POLAR_EXPRESS_COEFFS = [
    (8.156554524902461, -22.48329292557795, 15.878769915207462),
    (4.042929935166739, -2.808917465908714, 0.5000178451051316),
    (3.8916678022926607, -2.772484153217685, 0.5060648178503393),
    (3.285753657755655, -2.3681294933425376, 0.46449024233003106),
    (2.3465413258596377, -1.7097828382687081, 0.42323551169305323),
]

# Second coefficient table of the hybrid research fork: eight identical steps and two finishing ones
# (research/hybrid_attn/train.py:932-940)
DEEPSEEK_V4_COEFFS = [(3.4445, -4.7750, 2.0315)] * 8 + [(2.0, -1.5, 0.5)] * 2
NS_SCHEDULES = {"polar-express": POLAR_EXPRESS_COEFFS, "deepseek-v4": DEEPSEEK_V4_COEFFS}

c_void_p, c_int, c_long, c_float = _lib.c_void_p, _lib.c_int, _lib.ctypes.c_long, _lib.c_float


def _bf16(x: float) -> float:
    return float(torch.tensor(x, dtype=torch.float32).to(torch.bfloat16).float())


# ----------------------------------------------------------------------------- plain-PyTorch statements (oracle / CPU path)
def newton_schulz_ref(X: torch.Tensor, ns_steps: int, schedule: str = "polar-express") -> torch.Tensor:
    """X: [n, r, c] bf16 (already Frobenius-normalised). Returns the orthogonalised stack in bf16."""
    coeffs = NS_SCHEDULES[schedule]
    if X.size(-2) > X.size(-1):
        for a, b, c in coeffs[:ns_steps]:
            A = X.mT @ X
            X = a * X + X @ (b * A + c * (A @ A))
    else:
        for a, b, c in coeffs[:ns_steps]:
            A = X @ X.mT
            X = a * X + (b * A + c * (A @ A)) @ X
    return X


def muon_update_ref(G, M, S, momentum, beta2, ns_steps, row_norm=True, schedule="polar-express"):
    """Reference math of train.py:603-634 up to the variance-reduced update U (bf16). Updates M and S in place.
    G: [n, r, c] fp32 averaged gradient (consumed), M: momentum, S: second moment ([n,r,1] or [n,1,c]).
    `row_norm=False` is the tiny track's variant, which skips the MuonEq-R row normalisation (tiny/train.py:770-778).
    Matrices that received no gradient in a step (the reference's `active_mask`, tiny/train.py:773-809) are simply
    not passed in: with a zero mask that code leaves momentum, second moment and parameter of such a matrix
    untouched, which is what skipping it does."""
    mu = torch.tensor(momentum, dtype=G.dtype)     # the reference forms 1 - mu in the gradient dtype
    M.lerp_(G, (1 - mu).to(G.device))
    g = G.lerp_(M, mu.to(G.device))
    if row_norm:
        g /= g.float().norm(dim=-1, keepdim=True).clamp_min(1e-7).to(g.dtype)
    X = g.bfloat16()
    X = X / (X.norm(dim=(-2, -1), keepdim=True) * 1.02 + 1e-6)
    X = newton_schulz_ref(X, ns_steps, schedule)
    red_dim = -1 if G.size(-2) >= G.size(-1) else -2
    v_mean = X.float().square().mean(dim=red_dim, keepdim=True)
    red = X.size(red_dim)
    v_norm = (v_mean.sum(dim=(-2, -1), keepdim=True) * red).sqrt()
    # the reference casts beta2 to the (bf16) dtype of the orthogonalised update before forming 1 - beta2
    S.lerp_(v_mean.to(S.dtype), 1 - _bf16(beta2))
    step = S.clamp_min(1e-10).rsqrt()
    v_norm_new = ((v_mean * red) * step.float().square()).sum(dim=(-2, -1), keepdim=True).sqrt()
    final_scale = step * (v_norm / v_norm_new.clamp_min(1e-10))
    return X * final_scale.to(X.dtype)


def muon_apply_ref(P, U, lr_eff, wd):
    """Cautious weight decay + apply (train.py:635-639); lr and wd are rounded to bf16 as in the reference."""
    lr_b = _bf16(lr_eff)
    lrwd_b = _bf16(lr_b * _bf16(wd))
    g = U.float()
    upd = (lr_b * U).float() if U.dtype == torch.bfloat16 else (lr_b * g).bfloat16().float()
    mask = (g * P) >= 0
    P.sub_(upd + lrwd_b * P * mask)


def adamw_ref(p, grad, m, v, step, lr, b1, b2, eps, wd):
    """train.py:594-601"""
    p.mul_(1 - lr * wd)
    g = grad.to(p.dtype)
    m.lerp_(g, 1 - b1)
    v.lerp_(g.square(), 1 - b2)
    bias1 = 1 - b1 ** step
    bias2 = 1 - b2 ** step
    p.add_(m / ((v / bias2).sqrt() + eps), alpha=-(lr / bias1))


# ----------------------------------------------------------------------------- CUDA Newton-Schulz on the tcgen05 GEMM
class _NSWorkspace:
    def __init__(self, n, r, c, device):
        g = min(r, c)
        self.X2 = torch.empty((n, r, c), dtype=torch.bfloat16, device=device)
        self.A = torch.empty((n, g, g), dtype=torch.bfloat16, device=device)
        self.B = torch.empty((n, g, g), dtype=torch.bfloat16, device=device)


def newton_schulz_cuda(X: torch.Tensor, ns_steps: int, ws: _NSWorkspace, sym: bool = True,
                       schedule: str = "polar-express") -> torch.Tensor:
    """In: X [n, r, c] bf16. Three GEMMs per iteration; the gram and polynomial products are symmetric and only
    their upper-triangular tiles are computed; `aX + ...` and `bA + ...` ride in the epilogues."""
    n, r, c = X.shape
    tall = r > c
    src, dst = X, ws.X2[:n]
    A, B = ws.A[:n], ws.B[:n]
    for a_, b_, c_ in NS_SCHEDULES[schedule][:ns_steps]:
        if tall:
            gemm(src, src, out=A, a_mn=True, b_mn=True, sym=sym)                    # A = X^T X
            gemm(A, A, out=B, cin=A, alpha=c_, beta=b_, sym=sym)                    # B = bA + cA^2
            gemm(src, B, out=dst, cin=src, alpha=1.0, beta=a_)                      # X' = aX + X B
        else:
            gemm(src, src, out=A, sym=sym)                                          # A = X X^T
            gemm(A, A, out=B, cin=A, alpha=c_, beta=b_, sym=sym)
            gemm(B, src, out=dst, cin=src, b_mn=True, alpha=1.0, beta=a_)           # X' = aX + B X
        src, dst = dst, src
    return src


# ----------------------------------------------------------------------------- optimizer
class ShardedMuonAdamW:
    """`param_groups` is the list from `groups.build_param_groups`; the training loop rewrites lr / weight_decay /
    momentum in it every step exactly as with a torch optimizer."""

    def __init__(self, model, param_groups: List[dict], comm, use_cuda_kernels=None, wire_dtype: str = "bf16"):
        """`wire_dtype`: format in which gradients cross NVLink on the peer-memory path. "bf16": each rank rounds its
        accumulated fp32 gradients once into a bf16 copy that the owners read (half the bytes; the sum is formed in
        fp32); "fp32": the owners read the fp32 arenas directly. The torch.distributed path always reduces fp32."""
        self.model = model
        self.wire_dtype = wire_dtype
        # all-gather of the updates by multicast stores (needs a multicast mapping; SLOWRUN_PUSH_UPDATES=0 keeps the pull)
        self.push_updates = os.environ.get("SLOWRUN_PUSH_UPDATES", "1") != "0"
        self.sm_count = torch.cuda.get_device_properties(0).multi_processor_count if torch.cuda.is_available() else 0
        self.arena: ParamArena = model.arena
        self.param_groups = param_groups
        self.comm = comm
        self.rank, self.world = comm.rank, comm.world
        dev = model.get_device()
        self.cuda = dev.type == "cuda" if use_cuda_kernels is None else use_cuda_kernels
        self.device = dev
        self.state = {}
        self.step_count = 0
        self.fused = bool(getattr(comm, "fused", False)) and self.world > 1 and self.cuda and self.arena.symmetric
        self._inactive = set()      # ids of parameters that receive no gradient in the coming steps
        if self.arena.world_size != self.world:
            raise ValueError(f"arena was laid out for world size {self.arena.world_size}, comm has {self.world}")
        self._init_state()

    # ------------------------------------------------------------------ state
    def _init_state(self):
        dev, W = self.device, self.world
        for g in self.param_groups:
            if g["kind"] == "muon":
                ga = self.arena.groups[tuple(g["params"][0].shape)]
                r, c = ga.shape
                st = dict(arena=ga,
                          momentum=torch.zeros((ga.chunk, r, c), dtype=torch.float32, device=dev),
                          second=torch.zeros((ga.chunk, r, 1) if r >= c else (ga.chunk, 1, c), dtype=torch.float32, device=dev),
                          grad_chunk=torch.empty((ga.chunk, r, c), dtype=torch.float32, device=dev) if (W > 1 and not self.fused) else None,
                          U=(self.comm.alloc((ga.chunk, r, c), torch.bfloat16) if (self.fused and ga.W16 is not None)
                             else torch.zeros((ga.chunk, r, c), dtype=torch.bfloat16, device=dev)),
                          # gathered updates: symmetric on the peer-memory path, so that owners can push their chunk into
                          # every rank's copy through the multicast address
                          U_all=(self.comm.alloc((ga.n_pad, r, c), torch.bfloat16) if (self.fused and ga.W16 is not None)
                                 else (torch.empty((ga.n_pad, r, c), dtype=torch.bfloat16, device=dev) if W > 1 else None)))
                if self.fused and ga.W16 is not None and self.wire_dtype == "bf16" and c % 8 == 0:
                    st["G16"] = self.comm.alloc((ga.n_pad, r, c), torch.bfloat16)
                if self.cuda and ga.W16 is not None:
                    st["X"] = torch.empty((ga.chunk, r, c), dtype=torch.bfloat16, device=dev)
                    st["ws"] = _NSWorkspace(ga.chunk, r, c, dev)
                    ln = r if r >= c else c
                    st["scratch"] = torch.empty((3, ga.chunk, max(ln, 1)), dtype=torch.float32, device=dev)
                    st["sumsq"] = torch.empty(ga.chunk, dtype=torch.float32, device=dev)
                self.state[g["name"]] = st
            else:
                for p in g["params"]:
                    small = id(p) in self.arena.small_offsets
                    sharded = (not small) and W > 1 and p.shape[0] % W == 0
                    rows = p.shape[0] // W if sharded else p.shape[0]
                    shp = (rows,) + tuple(p.shape[1:])
                    self.state[id(p)] = dict(m=torch.zeros(shp, dtype=p.dtype, device=dev), v=torch.zeros(shp, dtype=p.dtype, device=dev),
                                             sharded=sharded, small=small, rows=rows)

    def num_owned(self, ga) -> int:
        return min(ga.chunk, max(0, ga.n - self.rank * ga.chunk))

    def set_inactive(self, params):
        """Declare parameters that get no gradient until further notice (layers a growing model does not run yet,
        research/universal_transformer/train.py:659-755; the `active_mask` of tiny/train.py:773-809). The step leaves
        their values and their optimizer state untouched. Pass an empty list to make everything active again."""
        self._inactive = {id(p) for p in params}

    def _active_runs(self, ga, first, count):
        """Maximal runs [a, b) of active matrices among stack slots first .. first + count - 1, as offsets from `first`."""
        if not self._inactive:
            return [(0, count)] if count > 0 else []
        runs, start = [], None
        for j in range(count):
            on = id(ga.params[first + j]) not in self._inactive
            if on and start is None:
                start = j
            if not on and start is not None:
                runs.append((start, j))
                start = None
        if start is not None:
            runs.append((start, count))
        return runs

    # ------------------------------------------------------------------ gradient source for AdamW params
    def _grad_of(self, p):
        if p is self.model.lm_head.weight:
            # CUDA ops accumulate the head gradient into the fp32 arena buffer; the plain-PyTorch path (CPU) leaves an
            # autograd-made .grad on a bf16 head instead
            if p.grad is not None and p.grad.data_ptr() != self.arena.head_grad.data_ptr():
                return p.grad
            return self.arena.head_grad
        return p.grad

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self):
        if getattr(self, "_prepulled", False):
            self._prepulled = False
            return self._step_fused(prepulled=True)
        if self.fused and not self._inactive:
            return self._step_fused_tuned()
        return self._step_library()

    @torch.no_grad()
    def _step_library(self):
        """The torch.distributed (NCCL / Gloo) formulation: reduce-scatter, owner update, all-gather of bf16 updates."""
        self.step_count += 1
        W, rank, comm = self.world, self.rank, self.comm
        gscale = 1.0 / W
        pending = []
        # phase 1: launch every gradient reduction
        small_h = comm.all_reduce_sum(self.arena.small_grads) if W > 1 else None
        for g in self.param_groups:
            if g["kind"] == "muon":
                st = self.state[g["name"]]
                ga = st["arena"]
                if W > 1 and st["grad_chunk"] is None:      # peer-memory job that runs this path (mode measurement)
                    r_, c_ = ga.shape
                    st["grad_chunk"] = torch.empty((ga.chunk, r_, c_), dtype=torch.float32, device=self.device)
                    if st["U_all"] is None:
                        st["U_all"] = torch.empty((ga.n_pad, r_, c_), dtype=torch.bfloat16, device=self.device)
                st["h"] = comm.reduce_scatter_sum(st["grad_chunk"], ga.G) if W > 1 else None
            else:
                for p in g["params"]:
                    st = self.state[id(p)]
                    if st["small"] or W == 1:
                        st["h"] = None
                        continue
                    grad = self._grad_of(p)
                    if st["sharded"]:
                        st["gslice"] = torch.empty((st["rows"],) + tuple(p.shape[1:]), dtype=grad.dtype, device=grad.device)
                        st["h"] = comm.reduce_scatter_sum(st["gslice"], grad)
                    else:
                        st["h"] = comm.all_reduce_sum(grad)
        # phase 2: compute per group, launch gathers
        if small_h is not None:
            small_h.wait()
        for g in self.param_groups:
            if g["kind"] == "muon":
                self._muon_compute(g, gscale, pending)
            else:
                self._adamw_compute(g, gscale, pending)
        # phase 3: finish gathers, apply matrix updates everywhere
        for item in pending:
            item()

    # ------------------------------------------------------------------ phase tracing (off unless `trace_phases` is set)
    def _mark(self, name):
        """With `self.trace_phases = True` every call records a CUDA event; `phase_report()` turns the list of one step
        into (phase, ms) pairs. Costs nothing when off."""
        if getattr(self, "trace_phases", False):
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._marks.append((name, ev))

    def phase_report(self):
        torch.cuda.synchronize()
        marks = getattr(self, "_marks", [])
        out = {}
        for (n0, e0), (n1, e1) in zip(marks[:-1], marks[1:]):
            out[n1] = out.get(n1, 0.0) + e0.elapsed_time(e1)
        return out

    # ------------------------------------------------------------------ which formulation of the step: measured
    TUNE_MODES = ("fused", "fused_two_streams", "library")
    TUNE_WARM, TUNE_TIMED = 2, 2       # per formulation: untimed steps (library collectives set themselves up lazily), timed steps

    def _run_mode(self, mode):
        if mode == "library":
            return self._step_library()
        self.overlap = mode == "fused_two_streams"
        return self._step_fused()

    def _step_fused_tuned(self):
        """`self.mode` is one of TUNE_MODES or "auto" (default). In "auto" the first twelve steps of the run try the three
        formulations in turn (two warm-up steps and two device-timed steps each: peer-memory kernels back to back,
        peer-memory kernels on two streams, the torch.distributed collectives), the maximum over ranks of the better
        timed step is compared and the fastest is kept for the rest of the run. All three compute the same update from the same state, so
        switching between steps is harmless. Setting `self.overlap` to True / False (older interface) pins the
        two-stream / one-stream peer-memory order."""
        mode = getattr(self, "mode", "auto")
        ov = getattr(self, "overlap", "auto")
        if mode == "auto" and ov != "auto":
            mode = "fused_two_streams" if ov else "fused"
        if mode != "auto":
            return self._run_mode(mode)
        if not hasattr(self, "_tune"):
            self._tune = []
        k = len(self._tune)
        per = self.TUNE_WARM + self.TUNE_TIMED
        cand = self.TUNE_MODES[k // per]
        timed = k % per >= self.TUNE_WARM
        if timed:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        try:
            self._run_mode(cand)
        finally:
            self.overlap = "auto"
        ms = float("inf")
        if timed:
            e1.record()
            e1.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float32, device=self.device)
            ms = float(self.comm.all_reduce_max(t).item())
        self._tune.append(ms)
        if len(self._tune) == per * len(self.TUNE_MODES):
            times = {m: min(self._tune[per * i:per * (i + 1)]) for i, m in enumerate(self.TUNE_MODES)}
            self.mode = min(times, key=times.get)
            self.tuned = {"ms": times, "mode": self.mode}

    @property
    def tuning_steps_left(self) -> int:
        """Optimizer steps until the measured choice among the step formulations is made (0 when nothing is being tuned)."""
        if not (self.fused and not self._inactive) or getattr(self, "mode", "auto") != "auto" or \
                getattr(self, "overlap", "auto") != "auto":
            return 0
        return (self.TUNE_WARM + self.TUNE_TIMED) * len(self.TUNE_MODES) - len(getattr(self, "_tune", []))

    # ------------------------------------------------------------------ pieces of the peer-memory step
    def _fast_groups(self):
        muon = [(g, self.state[g["name"]]) for g in self.param_groups if g["kind"] == "muon"]
        return [(g, st) for g, st in muon if "X" in st and st["arena"].W16 is not None]

    def _pack_wire(self, st, slot0, n):
        """Round this rank's fp32 gradients of slots [slot0, slot0 + n) into the bf16 wire buffer (no-op on an fp32 wire)."""
        if "G16" not in st or n <= 0:
            return
        ga = st["arena"]
        src, dst = ga.G[slot0:slot0 + n], st["G16"][slot0:slot0 + n]
        rc = _lib.fn("sr_cast_f32_to_bf16", [c_void_p, c_void_p, c_long, c_void_p])(src.data_ptr(), dst.data_ptr(), src.numel(),
                                                                                    _lib.stream_ptr())
        _lib.check_rc(rc, "sr_cast_f32_to_bf16")

    def _pull(self, g, st, slot0, n, shared_sms):
        """Owner side of the gradient reduce-scatter fused with the Muon prologue, for owned slots [slot0, slot0 + n) of
        the group (absolute slot numbers): sum over all ranks, momentum, Nesterov, row norm, bf16 Newton-Schulz input."""
        import ctypes
        if n <= 0:
            return
        ga, comm = st["arena"], self.comm
        r, c = ga.shape
        cvp = ctypes.c_void_p
        local = slot0 - self.rank * ga.chunk
        wire16 = "G16" in st
        src = st["G16"] if wire16 else ga.G
        rc = _lib.fn("sr_muon_pre_multi", [cvp, cvp, cvp, c_int, c_int, c_int, c_long, cvp, cvp, cvp, c_int, c_int, c_int, c_float,
                                           c_float, c_int, c_int, cvp, cvp])(
            ctypes.cast(comm.peer_ptrs(src), cvp), comm.multicast_ptr(src), ga.G.data_ptr(), int(wire16), self.world, self.rank,
            slot0 * r * c, st["momentum"][local:].data_ptr(), st["X"][local:].data_ptr(), st["sumsq"][local:].data_ptr(), n, r, c,
            float(g["momentum"]), 1.0 / self.world, int(bool(g.get("row_norm", True))), int(shared_sms),
            _lib.status_buffer(self.device).data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "sr_muon_pre_multi")

    # ------------------------------------------------------------------ gradient reduction under the backward pass
    def can_overlap_backward(self) -> bool:
        return bool(self.fused and not self._inactive and hasattr(self.model, "layer_done_hook") and self._fast_groups())

    def begin_backward_overlap(self):
        """Call before the forward pass of the LAST micro-batch of a step (run eagerly, not from a captured graph).
        While its backward pass walks down the network, every layer whose gradients have become final is released: this
        rank rounds them into the wire buffer and raises its progress counter on the backward stream; on a side stream
        the rank waits until all ranks have released that layer and pulls the matrices it owns (sum over ranks, momentum,
        Nesterov, row norm -> Newton-Schulz input). The arenas order each shape group by (layer mod world, layer), so
        every rank has something to pull every few layers. `finish_backward_overlap()` releases what is left; `step()`
        then starts from the pulled inputs."""
        if not self.can_overlap_backward():
            return False
        dev = self.device
        if getattr(self, "_ov_side", None) is None:
            self._ov_side = torch.cuda.Stream(device=dev)
            self._progress_count = 0
            # per layer: the runs of consecutive slots that hold its matrices, per fast group
            self._layer_runs = {}
            for g, st in self._fast_groups():
                ga = st["arena"]
                start = 0
                for s_ in range(1, ga.n + 1):
                    if s_ == ga.n or ga.layers[s_] != ga.layers[start]:
                        self._layer_runs.setdefault(ga.layers[start], []).append((g, st, start, s_ - start))
                        start = s_
        self._ov_top = max(k for k in self._layer_runs if k is not None)
        self._ov_next = self._ov_top          # highest layer not yet released
        self._ov_side.wait_stream(torch.cuda.current_stream(dev))
        self.model.layer_done_hook = self._on_layer_done
        self._ov_active = True
        return True

    def _on_layer_done(self, i):
        while self._ov_next > i:
            self._release_layer(self._ov_next)
            self._ov_next -= 1

    def _release_layer(self, L):
        runs = self._layer_runs.get(L, [])
        for g, st, slot0, n in runs:
            self._pack_wire(st, slot0, n)
        self._progress_count += 1
        value = self._progress_count
        self.comm.signal(value)
        with torch.cuda.stream(self._ov_side):
            self.comm.wait_for(value)
            for g, st, slot0, n in runs:
                ga = st["arena"]
                lo = max(slot0, self.rank * ga.chunk)
                hi = min(slot0 + n, self.rank * ga.chunk + self.num_owned(ga))
                self._pull(g, st, lo, hi - lo, shared_sms=True)

    def finish_backward_overlap(self):
        """Call after the backward pass returned: releases the layers no hook has released (the first ones)."""
        if not getattr(self, "_ov_active", False):
            return
        self.model.layer_done_hook = None
        while self._ov_next >= 0:
            self._release_layer(self._ov_next)
            self._ov_next -= 1
        if None in self._layer_runs:                                # matrices outside the layer stack, if any
            self._release_layer(None)
        self._ov_active = False
        self._prepulled = True

    # ------------------------------------------------------------------ fused peer-memory step
    @torch.no_grad()
    def _step_fused(self, prepulled: bool = False):
        """Same update as `step()`, with every collective replaced by a kernel that reads the peers' symmetric buffers
        and consumes the data in the same pass (csrc/comm_fused.cu), pipelined over two streams:

          side stream   barrier A (every rank's gradients are final) -> gradient pull + Muon prologue of every shape
                        group, then the AdamW row-slice pulls and updates -> per group, once its updates are final on
                        this rank: barrier B_g and the update pull fused with the cautious-weight-decay apply ->
                        last barrier, slice gathers of the sharded AdamW parameters
          main stream   small replicated parameters; per group, as soon as its pull has landed: Newton-Schulz and
                        the variance-reduction epilogue

        so NVLink traffic (pulls, applies) overlaps the Newton-Schulz GEMMs of the neighbouring groups. All
        device-side barriers are issued on the side stream, in the same order on every rank."""
        import ctypes
        self.step_count += 1
        W, rank, comm, arena = self.world, self.rank, self.comm, self.arena
        gscale = 1.0 / W
        head = self.model.lm_head.weight
        cvp = ctypes.c_void_p
        status_ptr = _lib.status_buffer(self.device).data_ptr()
        self._marks = []
        self._mark("start")
        main = torch.cuda.current_stream(self.device)
        if prepulled:
            side = self._ov_side   # the gradient pulls of this step are already queued there (begin_backward_overlap)
        elif getattr(self, "overlap", False) is True:
            if getattr(self, "_side", None) is None:
                self._side = torch.cuda.Stream(device=self.device)
            side = self._side
        else:
            side = main        # one stream: the same sequence, run back to back (every wait below is then a no-op)
        muon = [(g, self.state[g["name"]]) for g in self.param_groups if g["kind"] == "muon"]
        fast = self._fast_groups()
        slow = [(g, st) for g, st in muon if not ("X" in st and st["arena"].W16 is not None)]
        gathers = []

        def pull(i):
            """Side stream: gradient pull + Muon prologue of fast group i; returns the event that marks its end."""
            g, st = fast[i]
            ga = st["arena"]
            if not prepulled:
                self._pull(g, st, rank * ga.chunk, self.num_owned(ga), shared_sms=side is not main)
            ev = torch.cuda.Event()
            ev.record(side)
            return ev

        def adamw_big():
            """Side stream: row-slice pulls and updates of the large AdamW parameters (lm_head, wte, ...)."""
            for g in self.param_groups:
                if g["kind"] == "muon":
                    continue
                for p in g["params"]:
                    st = self.state[id(p)]
                    if st["small"]:
                        continue
                    grad = self._grad_of(p)
                    if st["sharded"]:
                        rows = st["rows"]
                        per_row = p.numel() // p.shape[0]
                        if "gslice32" not in st:
                            st["gslice32"] = torch.empty((rows,) + tuple(p.shape[1:]), dtype=torch.float32, device=self.device)
                        comm.reduce_from_peers(grad, rank * rows * per_row, st["gslice32"])
                        self._adamw_launch(p.data[rank * rows:(rank + 1) * rows], st["gslice32"], st["m"], st["v"], None, g, gscale)
                        gathers.append(p)
                    else:
                        if "gfull32" not in st:
                            st["gfull32"] = torch.empty(p.shape, dtype=torch.float32, device=self.device)
                        comm.reduce_from_peers(grad, 0, st["gfull32"])
                        shadow = arena.head_w16 if (p is head and arena.head_w16 is not None) else None
                        self._adamw_launch(p.data, st["gfull32"], st["m"], st["v"], shadow, g, gscale)

        side.wait_stream(main)
        with torch.cuda.stream(side):
            if not prepulled:
                for g, st in fast:                       # bf16 wire: round this rank's gradients once, before the barrier
                    self._pack_wire(st, 0, st["arena"].n)
            comm.device_barrier()                                                                  # A
            ev_a = torch.cuda.Event()
            ev_a.record(side)
            if side is main:
                self._mark("barrier_a")
            pull_done = [pull(i) for i in range(len(fast))]      # all pulls first: they gate the compute
            if side is main:
                self._mark("muon_pull_pre")
            adamw_big()
            if side is main:
                self._mark("adamw_big")
        # ---- main stream: small replicated parameters (one packed all-reduce read), then the per-group compute
        main.wait_event(ev_a)
        if side is not main:
            self._mark("barrier_a")
        if arena.small_grads.numel() > 0:
            if "small_sum" not in self.state:
                self.state["small_sum"] = torch.empty(arena.small_grads.numel(), dtype=torch.float32, device=self.device)
            small_sum = self.state["small_sum"]
            comm.reduce_from_peers(arena.small_grads, 0, small_sum)
            for g in self.param_groups:
                if g["kind"] != "muon":
                    smalls = [p for p in g["params"] if self.state[id(p)]["small"]]
                    if smalls:
                        self._adamw_small(g, smalls, small_sum, gscale)
        self._mark("adamw_small")
        for i, (g, st) in enumerate(fast):
            ga = st["arena"]
            r, c = ga.shape
            n_own = self.num_owned(ga)
            main.wait_event(pull_done[i])
            self._mark("wait_pull")
            if n_own > 0:
                sc = st["scratch"]
                Xo = newton_schulz_cuda(st["X"][:n_own], int(g["ns_steps"]), st["ws"],
                                        schedule=g.get("ns_schedule", "polar-express"))
                self._mark("newton_schulz")
                rc = _lib.fn("sr_muon_post", [c_void_p] * 5 + [c_int, c_int, c_int, c_float, c_void_p])(
                    Xo.data_ptr(), sc[0].data_ptr(), st["second"].data_ptr(), sc[1].data_ptr(), st["U"].data_ptr(),
                    n_own, r, c, _bf16(float(g["beta2"])), _lib.stream_ptr())
                _lib.check_rc(rc, "sr_muon_post")
                self._mark("muon_post")
            ev_post = torch.cuda.Event()
            ev_post.record(main)
            with torch.cuda.stream(side):
                side.wait_event(ev_post)
                lr_b = _bf16(float(g["lr"]) * max(1.0, r / c) ** 0.5)
                lrwd_b = _bf16(lr_b * _bf16(float(g["weight_decay"])))
                mc_all = comm.multicast_ptr(st["U_all"]) if self.push_updates else 0
                if mc_all:
                    # all-gather by push: the owner's chunk goes through the switch into every rank's U_all (one
                    # multimem store per 16 bytes), then every rank applies from its own memory
                    if n_own > 0:
                        rc = _lib.fn("sr_bcast_multi", [cvp, cvp, c_long, c_int, cvp, cvp])(
                            st["U"].data_ptr(), mc_all + rank * ga.chunk * r * c * 2, n_own * r * c * 2,
                            self.sm_count if side is not main else 0, status_ptr, _lib.stream_ptr())
                        _lib.check_rc(rc, "sr_bcast_multi")
                    comm.device_barrier()                                                          # B_g
                    rc = _lib.fn("sr_muon_apply_status", [cvp, cvp, cvp, c_long, c_float, c_float, cvp, cvp])(
                        ga.P.data_ptr(), st["U_all"].data_ptr(), ga.W16.data_ptr(), ga.P.numel(), lr_b, lrwd_b, status_ptr,
                        _lib.stream_ptr())
                    _lib.check_rc(rc, "sr_muon_apply_status")
                else:
                    comm.device_barrier()                                                          # B_g
                    rc = _lib.fn("sr_muon_apply_multi", [cvp, cvp, c_int, c_long, cvp, c_long, c_float, c_float, cvp, cvp])(
                        ga.P.data_ptr(), ctypes.cast(comm.peer_ptrs(st["U"]), cvp), W, ga.chunk * r * c, ga.W16.data_ptr(),
                        ga.P.numel(), lr_b, lrwd_b, status_ptr, _lib.stream_ptr())
                    _lib.check_rc(rc, "sr_muon_apply_multi")
        # ---- side stream: shape groups without the kernel path (no bf16 shadow), then the AdamW slice gathers
        side.wait_stream(main)
        with torch.cuda.stream(side):
            for g, st in slow:
                ga = st["arena"]
                r, c = ga.shape
                n_own = self.num_owned(ga)
                if n_own > 0:
                    tmp = torch.empty((n_own, r, c), dtype=torch.float32, device=self.device)
                    comm.reduce_from_peers(ga.G, rank * ga.chunk * r * c, tmp)
                    tmp.mul_(gscale)
                    st["U"][:n_own].copy_(muon_update_ref(tmp, st["momentum"][:n_own], st["second"][:n_own],
                                                          float(g["momentum"]), float(g["beta2"]), int(g["ns_steps"]),
                                                          bool(g.get("row_norm", True)), g.get("ns_schedule", "polar-express")))
            comm.device_barrier()                                                                  # last
            for g, st in slow:
                ga = st["arena"]
                r, c = ga.shape
                comm.all_gather(st["U_all"], st["U"], async_op=False)
                muon_apply_ref(ga.P, st["U_all"][:ga.n], float(g["lr"]) * max(1.0, r / c) ** 0.5, float(g["weight_decay"]))
            for p in gathers:
                comm.gather_slices(p.data)
                if p is head and arena.head_w16 is not None:
                    arena.head_w16.copy_(p.data)
        main.wait_stream(side)
        self._mark("join")

    def _adamw_small(self, grp, smalls, grads_flat, gscale):
        """One launch per run of parameters that are adjacent in the flat small-parameter buffer."""
        arena = self.arena
        segs = sorted(arena.small_offsets[id(p)] for p in smalls)
        merged = []
        for off, n in segs:
            if merged and merged[-1][0] + merged[-1][1] == off:
                merged[-1][1] += n
            else:
                merged.append([off, n])
        if "small_m" not in self.state:
            self.state["small_m"] = torch.zeros_like(arena.small_P)
            self.state["small_v"] = torch.zeros_like(arena.small_P)
        for off, n in merged:
            sl = slice(off, off + n)
            self._adamw_launch(arena.small_P[sl], grads_flat[sl], self.state["small_m"][sl], self.state["small_v"][sl],
                               None, grp, gscale)

    # ------------------------------------------------------------------ AdamW
    def _adamw_launch(self, p_t, g_t, m_t, v_t, shadow, grp, gscale):
        lr, wd = float(grp["lr"]), float(grp["weight_decay"])
        b1, b2 = grp["betas"]
        t = self.step_count
        if self.cuda:
            g32 = g_t if g_t.dtype == torch.float32 else g_t.float()
            rc = _lib.fn("sr_adamw", [c_void_p] * 5 + [c_long, c_int] + [c_float] * 8 + [c_void_p])(
                p_t.data_ptr(), g32.data_ptr(), m_t.data_ptr(), v_t.data_ptr(), _lib.ptr(shadow), p_t.numel(),
                int(p_t.dtype == torch.bfloat16), lr, wd, b1, b2, float(grp["eps"]), 1 - b1 ** t, 1 - b2 ** t, gscale,
                _lib.stream_ptr())
            _lib.check_rc(rc, "sr_adamw")
        else:
            adamw_ref(p_t, g_t.float() * gscale, m_t, v_t, t, lr, b1, b2, float(grp["eps"]), wd)
            if shadow is not None:
                shadow.copy_(p_t)

    def _adamw_compute(self, grp, gscale, pending):
        W, rank = self.world, self.rank
        arena = self.arena
        head = self.model.lm_head.weight
        smalls = [p for p in grp["params"] if self.state[id(p)]["small"] and id(p) not in self._inactive]
        if smalls:
            self._adamw_small(grp, smalls, arena.small_grads, gscale)
        for p in grp["params"]:
            st = self.state[id(p)]
            if st["small"]:
                continue
            if id(p) in self._inactive:
                if st.get("h") is not None:
                    st["h"].wait()
                continue
            if st.get("h") is not None:
                st["h"].wait()
            shadow_full = arena.head_w16 if (p is head and arena.head_w16 is not None) else None
            if st["sharded"]:
                rows = st["rows"]
                sl = slice(rank * rows, (rank + 1) * rows)
                p_slice = p.data[sl]
                self._adamw_launch(p_slice, st["gslice"], st["m"], st["v"], None, grp, gscale)
                h = self.comm.all_gather(p.data, p_slice)
                def fin(h=h, shadow_full=shadow_full, p=p):
                    h.wait()
                    if shadow_full is not None:
                        shadow_full.copy_(p.data)
                pending.append(fin)
            else:
                self._adamw_launch(p.data, self._grad_of(p), st["m"], st["v"], shadow_full, grp, gscale)

    # ------------------------------------------------------------------ Muon
    def _muon_compute(self, grp, gscale, pending):
        st = self.state[grp["name"]]
        ga = st["arena"]
        W, rank = self.world, self.rank
        r, c = ga.shape
        if st.get("h") is not None:
            st["h"].wait()
        n_own = self.num_owned(ga)
        G = st["grad_chunk"] if W > 1 else ga.G
        U = st["U"]
        mu, beta2, ns = float(grp["momentum"]), float(grp["beta2"]), int(grp["ns_steps"])
        row_norm = bool(grp.get("row_norm", True))
        first = rank * ga.chunk
        for a0, a1 in self._active_runs(ga, first, n_own):
            k = a1 - a0
            if self.cuda and "X" in st:
                X = st["X"][a0:a1]
                sc = st["scratch"]
                rc = _lib.fn("sr_muon_pre", [c_void_p] * 4 + [c_int, c_int, c_int, c_float, c_float, c_int, c_void_p])(
                    G[a0:a1].data_ptr(), st["momentum"][a0:a1].data_ptr(), X.data_ptr(), st["sumsq"].data_ptr(), k, r, c, mu,
                    gscale, int(row_norm), _lib.stream_ptr())
                _lib.check_rc(rc, "sr_muon_pre")
                Xo = newton_schulz_cuda(X, ns, st["ws"], schedule=grp.get("ns_schedule", "polar-express"))
                rc = _lib.fn("sr_muon_post", [c_void_p] * 5 + [c_int, c_int, c_int, c_float, c_void_p])(
                    Xo.data_ptr(), sc[0].data_ptr(), st["second"][a0:a1].data_ptr(), sc[1].data_ptr(), U[a0:a1].data_ptr(), k, r, c,
                    _bf16(beta2), _lib.stream_ptr())
                _lib.check_rc(rc, "sr_muon_post")
            else:
                g_own = G[a0:a1].mul(gscale) if gscale != 1.0 else G[a0:a1].clone()
                U[a0:a1].copy_(muon_update_ref(g_own, st["momentum"][a0:a1], st["second"][a0:a1], mu, beta2, ns, row_norm,
                                               grp.get("ns_schedule", "polar-express")))
        if self._inactive and n_own > 0:
            for j in range(n_own):                       # an inactive matrix contributes a zero update
                if id(ga.params[first + j]) in self._inactive:
                    U[j].zero_()
        lr_eff = float(grp["lr"]) * max(1.0, r / c) ** 0.5
        wd = float(grp["weight_decay"])
        if W > 1:
            h = self.comm.all_gather(st["U_all"], U)
        else:
            h = None

        def fin():
            if h is not None:
                h.wait()
            Uall = st["U_all"][:ga.n] if W > 1 else U[:ga.n]
            for a0, a1 in self._active_runs(ga, 0, ga.n):     # one run (everything) unless parameters were declared inactive
                Pr, Ur = ga.P[a0:a1], Uall[a0:a1]
                if self.cuda and ga.W16 is not None:
                    lr_b = _bf16(lr_eff)
                    lrwd_b = _bf16(lr_b * _bf16(wd))
                    rc = _lib.fn("sr_muon_apply", [c_void_p] * 3 + [c_long, c_float, c_float, c_void_p])(
                        Pr.data_ptr(), Ur.data_ptr(), ga.W16[a0:a1].data_ptr(), Pr.numel(), lr_b, lrwd_b, _lib.stream_ptr())
                    _lib.check_rc(rc, "sr_muon_apply")
                else:
                    muon_apply_ref(Pr, Ur, lr_eff, wd)
                    if ga.W16 is not None:
                        ga.W16[a0:a1].copy_(Pr)
        pending.append(fin)

    # ------------------------------------------------------------------ (de)serialisation of the owned state
    def state_dict(self):
        out = {"step_count": self.step_count, "groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}
        tensors = {}
        for g in self.param_groups:
            if g["kind"] == "muon":
                st = self.state[g["name"]]
                tensors[g["name"] + ".momentum"] = st["momentum"]
                tensors[g["name"] + ".second"] = st["second"]
            else:
                for i, p in enumerate(g["params"]):
                    st = self.state[id(p)]
                    if not st["small"]:
                        tensors[f"{g['name']}.{i}.m"] = st["m"]
                        tensors[f"{g['name']}.{i}.v"] = st["v"]
        if "small_m" in self.state:
            tensors["small_m"], tensors["small_v"] = self.state["small_m"], self.state["small_v"]
        out["tensors"] = {k: v.detach().cpu() for k, v in tensors.items()}
        return out

    def load_state_dict(self, sd):
        self.step_count = sd["step_count"]
        for g, saved in zip(self.param_groups, sd["groups"]):
            g.update(saved)
        t = sd["tensors"]
        for g in self.param_groups:
            if g["kind"] == "muon":
                st = self.state[g["name"]]
                st["momentum"].copy_(t[g["name"] + ".momentum"])
                st["second"].copy_(t[g["name"] + ".second"])
            else:
                for i, p in enumerate(g["params"]):
                    st = self.state[id(p)]
                    if not st["small"]:
                        st["m"].copy_(t[f"{g['name']}.{i}.m"])
                        st["v"].copy_(t[f"{g['name']}.{i}.v"])
        if "small_m" in t:
            self.state["small_m"] = t["small_m"].to(self.device)
            self.state["small_v"] = t["small_v"].to(self.device)
