"""Hybrid softmax / linear-attention GPT of the research fork (research/hybrid_attn/train.py).

Selected layers swap the softmax attention for a gated-delta-rule token mixer: `GatedDeltaNetAttention`
(research/hybrid_attn/train.py:375-510) or `KimiDeltaAttention` (:513-635). Module and parameter names are the
reference's, so a `{name: tensor}` checkpoint moves between the two. The rest of the network is the package's `GPT`
(U-Net skips, value projections on the remaining softmax layers, lambdas, layer replay); the softmax layers keep
running through the fused block node on a GPU. The state recurrence itself is `ops.linear_attention.gated_delta_rule`
(CUDA kernel forward on a GPU) where the reference calls flash-linear-attention.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import ModelConfig
from ..ops.linear_attention import gated_delta_rule
from .gpt import GPT

KDA_GATE_LOWER_BOUND = -5.0


@dataclass
class HybridSpec:
    """Which layers use linear attention and how (the --gdn-* / --linear-attn-type flags of the fork)."""
    layers: Optional[List[int]] = None        # None = all softmax
    kind: str = "gdn"                          # gdn | kda
    head_dim_mode: str = "param-matched"       # gdn: key head dim = value head dim / 2 ("param-matched") or equal ("square")
    no_conv: bool = False
    use_recurrent: bool = False                # token-by-token reference recurrence instead of the kernel / chunked form
    profile: bool = False


def auto_linear_layers(n_layer: int) -> List[int]:
    """The fork's default layout: softmax on the first layer, every 7th and the last; linear attention elsewhere
    (research/hybrid_attn/train.py:1440-1444)."""
    softmax = {0, 7, 14, 21, n_layer - 1}
    return [i for i in range(n_layer) if i not in softmax]


def parse_linear_layers(spec: str, n_layer: int) -> Optional[List[int]]:
    if spec == "none":
        return None
    if spec == "auto":
        return auto_linear_layers(n_layer)
    return [int(x) for x in spec.split(",") if x.strip()]


def _init_dt_bias(n):
    dt = torch.exp(torch.rand(n) * (math.log(0.1) - math.log(0.001)) + math.log(0.001)).clamp(min=1e-4)
    return dt + torch.log(-torch.expm1(-dt))          # inverse softplus


class _LinearAttentionBase(nn.Module):
    is_linear_attention = True
    use_iha = False
    use_key_offset = False
    conv_size = 4

    def _make_convs(self, key_dim, value_dim, no_conv):
        self.use_short_conv = not no_conv
        if self.use_short_conv:
            mk = lambda ch: nn.Conv1d(ch, ch, self.conv_size, padding=self.conv_size - 1, groups=ch, bias=False)
            self.q_conv, self.k_conv, self.v_conv = mk(key_dim), mk(key_dim), mk(value_dim)
        else:
            self.q_conv = self.k_conv = self.v_conv = None

    adamw_kind = "linear_attention"

    def adamw_scalar_params(self):
        """Small per-head / per-channel parameters, biases and the short convolutions: stepped by AdamW without weight
        decay, not by Muon (research/hybrid_attn/train.py:815-855)."""
        ps = [self.A_log, self.dt_bias]
        if hasattr(self, "beta_bias"):
            ps.append(self.beta_bias)
        if getattr(self.b_proj, "bias", None) is not None:
            ps.append(self.b_proj.bias)
        for conv in (self.q_conv, self.k_conv, self.v_conv):
            if conv is not None:
                ps += list(conv.parameters())
        return ps

    @staticmethod
    def _short_conv(x, conv):
        """Causal depth-wise convolution over time (kernel 4) followed by SiLU; SiLU alone without the convolution."""
        if conv is None:
            return F.silu(x)
        T = x.size(1)
        return F.silu(conv(x.transpose(1, 2).to(conv.weight.dtype))[:, :, :T].transpose(1, 2).to(x.dtype))

    def _section(self, name):
        return self.profiler.section(name) if self.profiler is not None else _NULL

    def _mix(self, q, k, v, g, beta):
        """q, k: [B, T, H, Dk] raw; normalises them (L2 over the key dim, q scaled by Dk^-1/2) and runs the recurrence."""
        Dk = q.size(-1)
        q = F.normalize(q.float(), dim=-1) * Dk ** -0.5
        k = F.normalize(k.float(), dim=-1)
        return gated_delta_rule(q.to(v.dtype), k.to(v.dtype), v, g, beta, impl="recurrent" if self.use_recurrent else "auto")


class _Null:
    def __enter__(self):
        return None

    def __exit__(self, *a):
        return False


_NULL = _Null()


def _lin(x, layer):
    return F.linear(x, layer.weight.to(x.dtype), None if layer.bias is None else layer.bias.to(x.dtype))


class GatedDeltaNetAttention(_LinearAttentionBase):
    """Gated DeltaNet: one log-decay per head from a Mamba-2 style gate, write strength beta in (0, 2) (values above 1
    flip the sign of the erased component), gated RMSNorm on the output."""

    def __init__(self, config: ModelConfig, spec: HybridSpec, layer_idx: int):
        super().__init__()
        d, H = config.n_embd, config.n_head
        self.num_heads = H
        self.head_v_dim = d // H
        self.head_k_dim = self.head_v_dim if spec.head_dim_mode == "square" else self.head_v_dim // 2
        self.key_dim, self.value_dim = H * self.head_k_dim, H * self.head_v_dim
        self.layer_idx, self.use_recurrent = layer_idx, spec.use_recurrent
        self.qk_proj = nn.Linear(d, 2 * self.key_dim, bias=False)
        self.vg_proj = nn.Linear(d, 2 * self.value_dim, bias=False)
        self.o_proj = nn.Linear(self.value_dim, d, bias=False)
        self.a_proj = nn.Linear(d, H, bias=False)
        self.b_proj = nn.Linear(d, H, bias=True)
        self.beta_bias = nn.Parameter(torch.linspace(-1.5, 1.5, H))
        self.A_log = nn.Parameter(torch.zeros(H))
        self.dt_bias = nn.Parameter(torch.zeros(H))
        self._make_convs(self.key_dim, self.value_dim, spec.no_conv)
        self.dropout = config.dropout
        self.profiler = None

    @torch.no_grad()
    def reset_parameters(self, s):
        for lin in (self.qk_proj, self.vg_proj, self.a_proj, self.b_proj):
            nn.init.uniform_(lin.weight, -s, s)
        nn.init.zeros_(self.o_proj.weight)
        nn.init.zeros_(self.b_proj.bias)
        self.beta_bias.copy_(torch.linspace(-1.5, 1.5, self.num_heads))      # half the heads start below beta = 1, half above
        self.A_log.copy_(torch.empty(self.num_heads).uniform_(2, 8).log())
        self.dt_bias.copy_(_init_dt_bias(self.num_heads))
        for conv in (self.q_conv, self.k_conv, self.v_conv):
            if conv is not None:
                nn.init.normal_(conv.weight, std=0.02)

    def forward(self, x):
        B, T, _ = x.shape
        H = self.num_heads
        with self._section("gdn/proj"):
            q, k = _lin(x, self.qk_proj).split(self.key_dim, dim=-1)
            v, g_out = _lin(x, self.vg_proj).split(self.value_dim, dim=-1)
        with self._section("gdn/conv"):
            q, k, v = self._short_conv(q, self.q_conv), self._short_conv(k, self.k_conv), self._short_conv(v, self.v_conv)
        q, k = q.reshape(B, T, H, self.head_k_dim), k.reshape(B, T, H, self.head_k_dim)
        v = v.reshape(B, T, H, self.head_v_dim)
        beta = torch.sigmoid(_lin(x, self.b_proj).float() + self.beta_bias.float()) * 2.0
        g = -self.A_log.float().exp() * F.softplus(_lin(x, self.a_proj).float() + self.dt_bias.float())
        with self._section("gdn/kernel"):
            o = self._mix(q, k, v, g, beta)
        with self._section("gdn/output"):
            o = F.rms_norm(o, (self.head_v_dim,)) * F.silu(g_out.reshape(B, T, H, self.head_v_dim))
        return _lin(o.reshape(B, T, self.value_dim), self.o_proj)


class KimiDeltaAttention(_LinearAttentionBase):
    """Kimi Delta Attention: a log-decay per key CHANNEL, produced by a low-rank projection and bounded below
    (g = lower_bound * sigmoid(exp(A_log) * (f(x) + dt_bias)), the "safe gate" form), beta in (0, 1), sigmoid output
    gate through a low-rank projection."""

    def __init__(self, config: ModelConfig, spec: HybridSpec, layer_idx: int):
        super().__init__()
        d, H = config.n_embd, config.n_head
        self.num_heads = H
        self.head_k_dim = self.head_v_dim = d // H
        self.key_dim, self.value_dim = H * self.head_k_dim, H * self.head_v_dim
        self.layer_idx, self.use_recurrent = layer_idx, spec.use_recurrent
        self.lower_bound = KDA_GATE_LOWER_BOUND
        self.q_proj = nn.Linear(d, self.key_dim, bias=False)
        self.k_proj = nn.Linear(d, self.key_dim, bias=False)
        self.v_proj = nn.Linear(d, self.value_dim, bias=False)
        self.f_proj = nn.Sequential(nn.Linear(d, self.head_v_dim, bias=False), nn.Linear(self.head_v_dim, self.key_dim, bias=False))
        self.b_proj = nn.Linear(d, H, bias=False)
        self.g_proj = nn.Sequential(nn.Linear(d, self.head_v_dim, bias=False), nn.Linear(self.head_v_dim, self.value_dim, bias=False))
        self.o_proj = nn.Linear(self.value_dim, d, bias=False)
        self.A_log = nn.Parameter(torch.zeros(H))
        self.dt_bias = nn.Parameter(torch.zeros(self.key_dim))
        self._make_convs(self.key_dim, self.value_dim, spec.no_conv)
        self.dropout = config.dropout
        self.profiler = None

    @torch.no_grad()
    def reset_parameters(self, s):
        for lin in (self.q_proj, self.k_proj, self.v_proj, self.f_proj[0], self.f_proj[1], self.b_proj, self.g_proj[0], self.g_proj[1]):
            nn.init.uniform_(lin.weight, -s, s)
        nn.init.zeros_(self.o_proj.weight)
        self.A_log.zero_()
        self.dt_bias.copy_(_init_dt_bias(self.key_dim))
        for conv in (self.q_conv, self.k_conv, self.v_conv):
            if conv is not None:
                nn.init.normal_(conv.weight, std=0.02)

    def forward(self, x):
        B, T, _ = x.shape
        H, Dk, Dv = self.num_heads, self.head_k_dim, self.head_v_dim
        with self._section("kda/proj"):
            q, k, v = _lin(x, self.q_proj), _lin(x, self.k_proj), _lin(x, self.v_proj)
            f = _lin(_lin(x, self.f_proj[0]), self.f_proj[1])
            beta = torch.sigmoid(_lin(x, self.b_proj).float())
            g_out = _lin(_lin(x, self.g_proj[0]), self.g_proj[1])
        with self._section("kda/conv"):
            q, k, v = self._short_conv(q, self.q_conv), self._short_conv(k, self.k_conv), self._short_conv(v, self.v_conv)
        q, k, v = q.reshape(B, T, H, Dk), k.reshape(B, T, H, Dk), v.reshape(B, T, H, Dv)
        raw = f.float().reshape(B, T, H, Dk) + self.dt_bias.float().view(H, Dk)
        g = self.lower_bound * torch.sigmoid(self.A_log.float().exp().view(H, 1) * raw)
        with self._section("kda/kernel"):
            o = self._mix(q, k, v, g, beta)
        with self._section("kda/output"):
            o = F.rms_norm(o, (Dv,)) * torch.sigmoid(g_out.reshape(B, T, H, Dv))
        return _lin(o.reshape(B, T, self.value_dim), self.o_proj)


class HybridGPT(GPT):
    def __init__(self, config: ModelConfig, spec: HybridSpec):
        super().__init__(config)
        self.hybrid = spec
        layers = sorted(set(spec.layers or []))
        if any(not 0 <= i < config.n_layer for i in layers):
            raise ValueError(f"linear-attention layer indices must lie in [0, {config.n_layer}), got {layers}")
        if spec.kind == "kda" and config.head_dim != 128:
            raise ValueError(f"kda layers are built for head_dim 128, got {config.head_dim}")
        if spec.kind not in ("gdn", "kda"):
            raise ValueError(f"unknown linear attention type {spec.kind!r}")
        cls = GatedDeltaNetAttention if spec.kind == "gdn" else KimiDeltaAttention
        for i in layers:
            self.transformer.h[i].attn = cls(config, spec, i)
            if str(i) in self.ve_projs:              # value residuals exist only on the softmax layers
                del self.ve_projs[str(i)]
        self.linear_layers = layers

    def set_profiler(self, profiler):
        for i in self.linear_layers:
            self.transformer.h[i].attn.profiler = profiler
