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
