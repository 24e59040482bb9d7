"""Command-line / import shim: `from gradient_select import run_gradient_selection` keeps working for scripts written
against the reference layout (unlimited/gradient_select.py); the implementation lives in
slowrun_b200/train/selection.py."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from slowrun_b200.train.selection import select_members  # noqa: E402


def run_gradient_selection(P_active, k_values, opt_steps=300, lr=0.5, weight_decay=0.0, grad_clip=1.0, eps=1e-12, seed=0):
    res = select_members(P_active, k_values, opt_steps, lr, weight_decay, grad_clip, eps, seed)
    out = {"_alpha": res.alpha}
    for k, s in res.by_k.items():
        out[k] = {"selected_local": s.members, "weights_renorm": s.weights, "fit_loss": s.fit_loss}
    return out
