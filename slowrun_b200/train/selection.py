"""Ensemble member selection by learned mixture weights.

Given P[m, t] = probability that candidate m assigns to the true token t of a held-out "fitness" slice, fit logits a
so that w = softmax(a) minimises mean_t -log(sum_m w_m P[m, t]) (AdamW on a, gradient clipping), then for every
requested K keep the K largest weights and renormalise them. Same objective, optimiser settings and tie-breaking
as the reference's selection step (unlimited/gradient_select.py:22-97).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Sequence

import torch


@dataclass
class Selection:
    k: int
    members: List[int]          # row indices into P, ascending
    weights: List[float]        # renormalised, sums to 1
    fit_loss: float             # in-sample NLL of the selected mixture


@dataclass
class SelectionResult:
    alpha: List[float]
    by_k: Dict[int, Selection] = field(default_factory=dict)


def mixture_nll(weights: torch.Tensor, P: torch.Tensor, eps: float = 1e-12) -> torch.Tensor:
    return -torch.log((weights @ P).clamp_min(eps)).mean()


def fit_mixture_logits(P: torch.Tensor, steps: int = 300, lr: float = 0.5, weight_decay: float = 0.0,
                       grad_clip: float = 1.0, eps: float = 1e-12, seed: int = 0) -> torch.Tensor:
    M = P.size(0)
    g = torch.Generator(device=P.device).manual_seed(seed)
    alpha = (1e-4 * torch.randn(M, device=P.device, generator=g)).float().requires_grad_(True)
    opt = torch.optim.AdamW([alpha], lr=lr, weight_decay=weight_decay)
    for _ in range(steps):
        opt.zero_grad(set_to_none=True)
        loss = mixture_nll(torch.softmax(alpha, dim=0), P, eps)
        loss.backward()
        if grad_clip and grad_clip > 0:
            torch.nn.utils.clip_grad_norm_([alpha], max_norm=grad_clip)
        opt.step()
    return alpha.detach()


def select_members(P: torch.Tensor, k_values: Sequence[int], steps: int = 300, lr: float = 0.5,
                   weight_decay: float = 0.0, grad_clip: float = 1.0, eps: float = 1e-12, seed: int = 0) -> SelectionResult:
    """P: [M, N] float tensor. Returns the learned logits and, per K, the chosen members with their weights."""
    M = P.size(0)
    if M == 0:
        return SelectionResult(alpha=[])
    alpha = fit_mixture_logits(P.float(), steps, lr, weight_decay, grad_clip, eps, seed)
    w = torch.softmax(alpha, dim=0)
    res = SelectionResult(alpha=[float(a) for a in alpha.cpu()])
    for k in k_values:
        kk = min(int(k), M)
        idx = torch.topk(w, k=kk).indices.sort().values
        wk = w[idx] / w[idx].sum().clamp_min(eps)
        with torch.no_grad():
            fl = float(mixture_nll(wk, P[idx].float(), eps))
        res.by_k[int(k)] = Selection(k=int(k), members=idx.cpu().tolist(), weights=[float(x) for x in wk.cpu()], fit_loss=fl)
    return res
