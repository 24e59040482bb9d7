"""Loads pieces of the reference scripts as a CPU oracle for parity tests.

The reference scripts run their whole training at import, so tests cut out the self-contained sections (model,
optimizer math, loader, schedules) by their banner comments and exec them with the few globals they read. The
source tree is looked up at baseline/_ref (the copy that travels with the repo), then at the directory named by the
environment variable SLOWRUN_REFERENCE_DIR; tests that need it are skipped when neither exists.
"""
import math
import os
import types
from functools import partial
from dataclasses import dataclass
from types import SimpleNamespace

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def ref_root():
    for p in (os.path.join(ROOT, "baseline", "_ref"), os.environ.get("SLOWRUN_REFERENCE_DIR")):
        if p and os.path.isfile(os.path.join(p, "train.py")):
            return p
    return None


def _section(src: str, start_marker: str, end_marker: str) -> str:
    a = src.index(start_marker)
    b = src.index(end_marker, a)
    return src[a:b]


def _sdpa_attention(q, k, v, causal=True, window_size=(-1, -1), softmax_scale=None):
    """(B,T,H,D) causal sliding-window attention with the flash-attn window convention (keys i-left..i)."""
    B, T, H, D = q.shape
    q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    w = window_size[0]
    if w < 0 or w >= T:
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=softmax_scale)
    else:
        i = torch.arange(T).unsqueeze(1)
        j = torch.arange(T).unsqueeze(0)
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=(j <= i) & ((i - j) <= w), scale=softmax_scale)
    return y.transpose(1, 2)


def load_limited(n_layer=4, n_embd=128, n_head=4, seq_len=64, mtp_weight=0.3, iha=True, logit_cap=10.0):
    """Namespace holding the limited-track GPT, optimizer functions and DataLoader of the reference (CPU)."""
    root = ref_root()
    if root is None:
        return None
    src = open(os.path.join(root, "train.py")).read()
    model_src = _section(src, "@dataclass\nclass GPTConfig", "# =============================================================================\n# Optimizer")
    opt_src = _section(src, "# Polar Express coefficients", "# =============================================================================\n# Dataloader")
    opt_src = opt_src.replace("@torch.compile(dynamic=False, fullgraph=True)\n", "")
    loader_src = _section(src, "class DataLoader:", "# =============================================================================\n# Loss evaluation")
    args = SimpleNamespace(mtp_weight=mtp_weight, iha_lr=0.02)
    ns = dict(torch=torch, nn=nn, F=F, np=np, math=math, dataclass=dataclass, partial=partial, SimpleNamespace=SimpleNamespace,
              args=args, MAX_SEQ_LEN=seq_len, DEPTH=n_layer, N_HEAD=n_head, N_EMBD=n_embd, WINDOW_PATTERN="SSSL",
              LOGIT_CAP=logit_cap, BOS_ID=50256, dist=torch.distributed, Tensor=torch.Tensor,
              print0=lambda *a, **k: None, get_dist_info=lambda: (False, 0, 0, 1),
              flash_attn=SimpleNamespace(flash_attn_func=_sdpa_attention),
              UNEMBEDDING_LR=0.002, EMBEDDING_LR=0.15, SCALAR_LR=0.1, MATRIX_LR=0.04, WEIGHT_DECAY=1.3,
              ADAM_BETAS=(0.8, 0.95))
    exec(model_src, ns)
    exec(opt_src, ns)
    exec(loader_src, ns)
    return SimpleNamespace(**ns)


def load_unlimited_loaders():
    """The data-loading section of the reference's unlimited script (unlimited/train.py:758-965): DataLoader,
    DDPValLoader and the fitness carve, on CPU."""
    root = ref_root()
    if root is None:
        return None
    src = open(os.path.join(root, "unlimited", "train.py")).read()
    sec = _section(src, "# Data loading (flat tokens + doc_starts format", "# =============================================================================\n# Evaluation helpers")
    ns = dict(torch=torch, np=np, math=math)
    exec(sec, ns)
    return SimpleNamespace(**ns)


def load_tiny_optimizer():
    """The optimizer section of the reference's tiny script (tiny/train.py:748-946): its Muon step without row
    normalisation and with the active mask, run eagerly on CPU."""
    root = ref_root()
    if root is None:
        return None
    src = open(os.path.join(root, "tiny", "train.py")).read()
    sec = _section(src, "# Polar Express coefficients for orthogonalization", "# =============================================================================\n# Dataloader")
    sec = sec.replace("@torch.compile(dynamic=False, fullgraph=True)\n", "")
    ns = dict(torch=torch, dist=torch.distributed, Tensor=torch.Tensor)
    exec(sec, ns)
    return SimpleNamespace(**ns)


class _TinyLossOracle(torch.autograd.Function):
    """fp32 statement of the reference's fused loss (tiny/cuda_kernels.py:125-414) without the fp8 quantisation: per-row
    loss sum_k w_k (lse - z[target[r + k]]) over the flattened batch, and the gradient exactly as its kernel forms it
    (S_w p minus the weights of the targets that coincide with a column, times 1 - tanh^2; dW scaled by the mean of the
    incoming gradient)."""

    @staticmethod
    def forward(ctx, x, targets, mtp_weights, w, x_s, w_s, grad_s, grad_scale, cap=15.0):
        xf, wf = x.float(), w.float()
        t = torch.tanh(xf @ wf / cap)
        z = cap * t
        lse = torch.logsumexp(z, dim=-1)
        n = x.size(0)
        losses = torch.zeros(n)
        coef = torch.zeros_like(z)
        for k in range(mtp_weights.numel()):
            rows = torch.arange(0, n - k)
            tg = targets[rows + k]
            ok = (tg >= 0) & (tg < z.size(1))
            losses[rows[ok]] += mtp_weights[k] * (lse[rows[ok]] - z[rows[ok], tg[ok]])
            coef[rows[ok], tg[ok]] += mtp_weights[k]
        p = torch.exp(z - lse[:, None])
        gz = (mtp_weights.sum() * p - coef) * (1 - t * t)
        ctx.save_for_backward(gz, xf, wf)
        ctx.dt = (x.dtype, w.dtype)
        return losses

    @staticmethod
    def backward(ctx, go):
        gz, xf, wf = ctx.saved_tensors
        gx = (gz @ wf.t()) * go[:, None]
        gw = (xf.t() @ gz) * go.mean()
        return gx.to(ctx.dt[0]), None, None, gw.to(ctx.dt[1]), None, None, None, None, None


class _Done:
    def wait(self):
        return None

    def get_future(self):
        return self


class _OneRankDist:
    """Stand-in for torch.distributed with a single rank: every collective is a copy."""
    ReduceOp = SimpleNamespace(AVG="avg", SUM="sum")

    @staticmethod
    def get_rank():
        return 0

    @staticmethod
    def get_world_size():
        return 1

    @staticmethod
    def all_reduce(t, op=None, async_op=False):
        return _Done()

    @staticmethod
    def reduce_scatter_tensor(out, inp, op=None, async_op=False):
        out.copy_(inp.reshape(out.shape))
        return _Done()

    @staticmethod
    def all_gather_into_tensor(out, inp, async_op=False):
        if out.data_ptr() != inp.data_ptr():
            out.copy_(inp.reshape(out.shape))
        return _Done()


def load_tiny(n_layer=4, n_embd=256, n_head=2, seq_len=64, num_iterations=2):
    """Namespace holding the tiny-track GPT and optimizer of the reference (tiny/train.py:378-946) on CPU: attention
    through SDPA, the fused fp8 loss replaced by its fp32 statement above."""
    root = ref_root()
    if root is None:
        return None
    src = open(os.path.join(root, "tiny", "train.py")).read()
    model_src = _section(src, "@dataclass\nclass GPTConfig", "# =============================================================================\n# Optimizer")
    opt_src = _section(src, "# Polar Express coefficients for orthogonalization", "# =============================================================================\n# Dataloader")
    opt_src = opt_src.replace("@torch.compile(dynamic=False, fullgraph=True)\n", "")
    ns = dict(torch=torch, nn=nn, F=F, np=np, math=math, dataclass=dataclass, partial=partial, SimpleNamespace=SimpleNamespace,
              MAX_SEQ_LEN=seq_len, DEPTH=n_layer, N_HEAD=n_head, N_EMBD=n_embd, WINDOW_PATTERN="SSSL", NUM_ITERATIONS=num_iterations,
              TRAIN_BACKPROP_ITERATIONS=1, BOS_ID=50256, dist=_OneRankDist, Tensor=torch.Tensor,
              print0=lambda *a, **k: None, get_dist_info=lambda: (False, 0, 0, 1),
              flash_attn=SimpleNamespace(flash_attn_func=_sdpa_attention),
              FusedSoftcappedCrossEntropy=_TinyLossOracle, CE_KERNEL_VOCAB_SIZE=50304,
              MTP_X_S=100 / 448, MTP_W_S=1.6 / 448, MTP_GRAD_S=0.75 / 448,
              UNEMBEDDING_LR=0.001 * 0.8, EMBEDDING_LR=0.15 * 0.8, SCALAR_LR=0.25 * 0.8, MATRIX_LR=0.04 * 0.8, WEIGHT_DECAY=0.8,
              ADAM_BETAS=(0.8, 0.95))
    exec(model_src, ns)
    exec(opt_src, ns)
    return SimpleNamespace(**ns)
