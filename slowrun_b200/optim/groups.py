"""Parameter grouping: which parameters Muon orthogonalises, which AdamW steps, with which learning rates.

Same membership, order and hyper-parameters as the reference's `setup_optimizer` (limited: train.py:461-512,
tiny: tiny/train.py:627-664). Muon groups are one per distinct matrix shape, in sorted shape order, members in
module registration order — the order also fixes which rank owns which matrix.
"""
from __future__ import annotations

from typing import List

import torch

from ..config import TrainConfig


def _iha_params(model):
    if hasattr(model, "iha_params"):
        return model.iha_params()
    out = []
    for block in model.all_blocks():
        a = block.attn
        if a.use_iha:
            out += [a.q_mix, a.k_mix]
            if a.iha_mix_v:
                out.append(a.v_mix)
    return out


def adamw_flagged_params(model, kind=None) -> List[torch.nn.Parameter]:
    """Parameters inside the blocks that their module hands to AdamW through `adamw_scalar_params()` (per-head decays,
    biases and short convolutions of the linear-attention layers, research/hybrid_attn/train.py:815-855; learnable norm
    weights of the universal transformer). `kind` filters by the module's `adamw_kind`."""
    out = []
    for mod in model.modules():
        if hasattr(mod, "adamw_scalar_params") and (kind is None or mod.adamw_kind == kind):
            out += mod.adamw_scalar_params()
    return out


def muon_matrix_params(model) -> List[torch.nn.Parameter]:
    """Every parameter that the reference hands to Muon, in its order."""
    if hasattr(model, "muon_matrix_params"):
        return model.muon_matrix_params()
    flagged = {id(p) for p in adamw_flagged_params(model)}
    if model.config.attn_gate_adamw:
        gate_ids = {id(b.attn.attn_gate.weight) for b in model.transformer.h}
        ps = list(model.transformer.h.parameters()) + list(model.ve_projs.parameters())
        return [p for p in ps if id(p) not in gate_ids and id(p) not in flagged]
    iha_ids = {id(p) for p in _iha_params(model)} | flagged
    ps = [p for p in model.transformer.h.parameters() if id(p) not in iha_ids] + list(model.ve_projs.parameters())
    if model.mtp_weight > 0:
        ps += [p for p in list(model.mtp_block.parameters()) + list(model.mtp_proj.parameters()) if id(p) not in iha_ids]
    return ps


def muon_shape_groups(model):
    ps = muon_matrix_params(model)
    return [(shape, [p for p in ps if p.shape == shape]) for shape in sorted({p.shape for p in ps})]


def build_param_groups(model, cfg: TrainConfig):
    lrs = cfg.lrs
    wd = cfg.weight_decay
    betas = tuple(cfg.adam_betas)
    A = dict(kind="adamw", eps=1e-10)
    groups = [
        dict(A, name="lm_head", params=[model.lm_head.weight], lr=lrs["unembedding"], betas=betas, weight_decay=wd),
        dict(A, name="wte", params=list(model.transformer.wte.parameters()), lr=lrs["embedding"], betas=betas, weight_decay=wd),
        dict(A, name="resid", params=[model.resid_lambdas], lr=lrs["scalar"] * 0.01, betas=betas, weight_decay=0.0),
        dict(A, name="x0", params=[model.x0_lambdas], lr=lrs["scalar"], betas=(0.96, 0.95), weight_decay=0.0),
        dict(A, name="skip", params=[model.skip_weights], lr=lrs["scalar"] * 0.01, betas=betas, weight_decay=0.0),
    ]
    if model.config.attn_gate_adamw:
        gates = [b.attn.attn_gate.weight for b in model.transformer.h]
        groups.append(dict(A, name="attn_gate", params=gates, lr=lrs["scalar"], betas=(0.9, 0.99), weight_decay=0.0))
    else:
        iha = _iha_params(model)
        if iha:
            groups.append(dict(A, name="iha", params=iha, lr=cfg.iha_lr, betas=betas, weight_decay=0.0))
    # learnable XSA strengths (tiny/train.py:653-655); available to every track when xsa_mode is on
    if model.config.xsa_mode != "off" and hasattr(model, "xsa_alphas"):
        groups.append(dict(A, name="xsa", params=[model.xsa_alphas], lr=lrs["scalar"], betas=(0.9, 0.95), weight_decay=0.0))
    norms = adamw_flagged_params(model, "norm")
    others = adamw_flagged_params(model, "linear_attention")
    if norms:       # learnable norm weights of the universal transformer (research/universal_transformer/train.py:511)
        groups.append(dict(A, name="norms", params=norms, lr=lrs["scalar"], betas=betas, weight_decay=0.0))
    if others:      # decays, biases and short convolutions of linear-attention layers (research/hybrid_attn/train.py:852-854)
        groups.append(dict(A, name="block_scalars", params=others, lr=lrs["scalar"], betas=(0.9, 0.99), weight_decay=0.0))
    if getattr(model, "mtp_head", None) is not None:
        groups.append(dict(A, name="mtp_head", params=[model.mtp_head.weight], lr=lrs["unembedding"], betas=betas, weight_decay=wd))
    # MuonEq-R row normalisation of the Nesterov gradient: every track but tiny (train.py:611-613 vs tiny/train.py:770-778);
    # the hybrid fork makes it a switch (--no-muon-eq-r) and offers a second Newton-Schulz coefficient table
    row_norm = cfg.track != "tiny" and bool(getattr(cfg, "muon_eq_r", True))
    ns_schedule = getattr(cfg, "muon_ns_schedule", "polar-express")
    from .muon_adamw import NS_SCHEDULES
    ns_steps = cfg.ns_steps if ns_schedule == "polar-express" else len(NS_SCHEDULES[ns_schedule])
    for shape, ps in muon_shape_groups(model):
        groups.append(dict(kind="muon", name=f"muon{tuple(shape)}", params=ps, lr=lrs["matrix"], momentum=cfg.muon_momentum,
                           ns_steps=ns_steps, beta2=0.95, weight_decay=wd, row_norm=row_norm, ns_schedule=ns_schedule))
    for g in groups:
        g["initial_lr"] = g["lr"]
        g["initial_wd"] = g["weight_decay"]
    return groups
