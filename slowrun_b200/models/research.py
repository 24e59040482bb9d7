"""Research model variants of the reference repository, as plain-PyTorch modules (autograd, any device):

* `UniversalGPT` — the universal-transformer fork (research/universal_transformer/train.py:221-330, 432-437,
  530-584): each half of the U-Net shares TWO attention modules and ONE SwiGLU MLP (hidden 8d) across all of its
  layers; what is per-layer are learnable RMSNorms (weight + bias) for the attention inputs, q, k and the MLP input,
  the value / attention gates, lambdas and value projections. The number of active layers grows during training
  (`--depth-schedule "0:10,1533:20"`), new layers being inserted towards the middle of the U-Net.
* `GatedDeltaNetAttention` — the linear-attention block of the hybrid fork (research/hybrid_attn/train.py:375-635):
  gated delta rule S_t = a_t S_{t-1} (I - b_t k_t k_t^T) + b_t v_t k_t^T, o_t = S_t q_t, with optional short
  depth-wise convolutions on q/k/v and an output gate. The reference calls flash-linear-attention's Triton kernels;
  this is the recurrence itself (chunk-free), the numerics oracle for a future kernel.

These models reuse the GEMM-backed `ops.linear` path only through `torch.nn.functional.linear`; they are capability
surface, not the tuned flagship.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as ops
from .gpt import Rotary, has_ve


# =============================================================================== universal transformer
@dataclass
class UniversalConfig:
    sequence_len: int = 2048
    vocab_size: int = 50257
    n_layer: int = 20            # maximum depth
    n_head: int = 8
    n_embd: int = 1024
    window_pattern: str = "SSSL"
    dropout: float = 0.0
    stoch_depth: float = 0.05
    logit_cap: float = 10.0
    depth_schedule: str = "0:10,1533:20"


def parse_depth_schedule(spec: str) -> List[Tuple[int, int]]:
    """'0:10,1533:20' -> [(0, 10), (1533, 20)]: from step s on, run d layers (d even, non-decreasing)."""
    out = []
    for part in spec.split(","):
        s, d = part.split(":")
        out.append((int(s), int(d)))
    out.sort()
    assert out and out[0][0] == 0 and all(d % 2 == 0 for _, d in out)
    assert all(a[1] <= b[1] for a, b in zip(out, out[1:])), "depth may only grow"
    return out


def depth_at_step(schedule: List[Tuple[int, int]], step: int) -> int:
    d = schedule[0][1]
    for s, dd in schedule:
        if step >= s:
            d = dd
    return d


class LearnedRMSNorm(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.bias = nn.Parameter(torch.zeros(dim))

    def forward(self, x):
        return F.rms_norm(x, (x.size(-1),), self.weight.to(x.dtype)) + self.bias.to(x.dtype)


class SharedAttention(nn.Module):
    """Projection weights shared by all layers of one U-Net half; norms and gates come from the calling layer."""

    def __init__(self, c: UniversalConfig):
        super().__init__()
        d = c.n_embd
        self.n_head, self.head_dim = c.n_head, d // c.n_head
        self.c_q, self.c_k, self.c_v = (nn.Linear(d, d, bias=False) for _ in range(3))
        self.c_proj = nn.Linear(d, d, bias=False)
        self.dropout = c.dropout

    def forward(self, x, ve, cos_sin, window, q_norm, k_norm, ve_gate, attn_gate):
        B, T, _ = x.shape
        H, D = self.n_head, self.head_dim
        q = self.c_q(x).view(B, T, H, D)
        k = self.c_k(x).view(B, T, H, D)
        v = self.c_v(x).view(B, T, H, D)
        if ve is not None and ve_gate is not None:
            v = v + (2 * torch.sigmoid(ve_gate)).unsqueeze(-1) * ve.view(B, T, H, D)
        cos, sin = cos_sin
        d2 = D // 2

        def rot(t):
            t1, t2 = t[..., :d2], t[..., d2:]
            return torch.cat([t1 * cos + t2 * sin, t1 * (-sin) + t2 * cos], 3)
        q, k = q_norm(rot(q)), k_norm(rot(k))
        y = ops.attention_ref(q, k, v, window[0], None)
        y = y * torch.sigmoid(attn_gate).unsqueeze(-1)
        return F.dropout(self.c_proj(y.reshape(B, T, H * D)), self.dropout, self.training)


class SharedMLP(nn.Module):
    def __init__(self, c: UniversalConfig):
        super().__init__()
        h = 8 * c.n_embd
        self.c_gate = nn.Linear(c.n_embd, h, bias=False)
        self.c_fc = nn.Linear(c.n_embd, h, bias=False)
        self.c_proj = nn.Linear(h, c.n_embd, bias=False)
        self.dropout = c.dropout

    def forward(self, x):
        return F.dropout(self.c_proj(F.silu(self.c_gate(x)) * self.c_fc(x)), self.dropout, self.training)


class LayerParams(nn.Module):
    """Everything that is NOT shared: per-layer norms and gates."""

    def __init__(self, c: UniversalConfig, layer_idx: int):
        super().__init__()
        D = c.n_embd // c.n_head
        self.attn_norms = nn.ModuleList([LearnedRMSNorm(c.n_embd) for _ in range(2)])
        self.mlp_norm = LearnedRMSNorm(c.n_embd)
        self.q_norms = nn.ModuleList([LearnedRMSNorm(D) for _ in range(2)])
        self.k_norms = nn.ModuleList([LearnedRMSNorm(D) for _ in range(2)])
        ve = has_ve(layer_idx, c.n_layer)
        self.ve_gates = nn.ModuleList([nn.Linear(32, c.n_head, bias=False) if ve else nn.Identity() for _ in range(2)])
        self.attn_gates = nn.ModuleList([nn.Linear(12, c.n_head, bias=False) for _ in range(2)])
        self.drop_prob = c.stoch_depth * (layer_idx / max(c.n_layer - 1, 1))


class UniversalGPT(nn.Module):
    def __init__(self, c: UniversalConfig):
        super().__init__()
        self.config = c
        L = c.n_layer
        assert L % 2 == 0
        pv = ((c.vocab_size + 63) // 64) * 64
        self.transformer = nn.ModuleDict({"wte": nn.Embedding(pv, c.n_embd),
                                          "h": nn.ModuleList([LayerParams(c, i) for i in range(L)])})
        self.encoder_attns = nn.ModuleList([SharedAttention(c) for _ in range(2)])
        self.decoder_attns = nn.ModuleList([SharedAttention(c) for _ in range(2)])
        self.encoder_mlp, self.decoder_mlp = SharedMLP(c), SharedMLP(c)
        self.lm_head = nn.Linear(c.n_embd, pv, bias=False)
        self.resid_lambdas = nn.Parameter(torch.ones(L))
        self.x0_lambdas = nn.Parameter(torch.full((L,), 0.1))
        self.ve_projs = nn.ModuleDict({str(i): nn.Linear(c.n_embd, c.n_embd, bias=False) for i in range(L) if has_ve(i, L)})
        self.max_n_layer, self.max_encoder_layers = L, L // 2
        self.skip_weights = nn.Parameter(torch.ones(L // 2))
        self.rotary = Rotary(c.n_embd // c.n_head, c.sequence_len * 10)
        long_w, short_w = c.sequence_len, c.sequence_len // 2
        pat = c.window_pattern.upper()
        self.window_sizes = [((long_w if pat[i % len(pat)] == "L" else short_w), 0) for i in range(L)]
        self.window_sizes[-1] = (long_w, 0)
        self.schedule = parse_depth_schedule(c.depth_schedule)
        self.set_active_layers(self.schedule[0][1])
        self.init_weights()

    @torch.no_grad()
    def init_weights(self):
        c = self.config
        s = 3 ** 0.5 * c.n_embd ** -0.5
        nn.init.normal_(self.transformer.wte.weight, std=1.0)
        nn.init.normal_(self.lm_head.weight, std=0.001)
        for m in list(self.encoder_attns) + list(self.decoder_attns):
            for lin in (m.c_q, m.c_k, m.c_v):
                nn.init.uniform_(lin.weight, -s, s)
            nn.init.zeros_(m.c_proj.weight)
        for m in (self.encoder_mlp, self.decoder_mlp):
            nn.init.uniform_(m.c_gate.weight, -s, s)
            nn.init.uniform_(m.c_fc.weight, -s, s)
            nn.init.zeros_(m.c_proj.weight)
        for p in self.ve_projs.values():
            nn.init.uniform_(p.weight, -s, s)
        for blk in self.transformer.h:
            for g in list(blk.ve_gates) + list(blk.attn_gates):
                if isinstance(g, nn.Linear):
                    nn.init.zeros_(g.weight)
        self.rotary.reset()

    def set_active_layers(self, n_layer: int):
        """Run only `n_layer` layers: the first n/2 encoder layers and the last n/2 decoder layers, so growth adds
        layers next to the middle of the U-Net."""
        assert n_layer % 2 == 0 and 0 < n_layer <= self.max_n_layer
        self.active_n_layer = n_layer
        self.active_encoder_layers = n_layer // 2
        self.active_decoder_start = self.max_n_layer - n_layer // 2

    def apply_depth_schedule(self, step: int) -> bool:
        d = depth_at_step(self.schedule, step)
        changed = d != self.active_n_layer
        if changed:
            self.set_active_layers(d)
        return changed

    def _run_layer(self, x, x0, cos_sin, i, attns, mlp):
        blk = self.transformer.h[i]
        x = self.resid_lambdas[i] * x + self.x0_lambdas[i] * x0
        ve = self.ve_projs[str(i)](x0) if str(i) in self.ve_projs else None
        x_in = x
        for attn, an, qn, kn, vg, ag in zip(attns, blk.attn_norms, blk.q_norms, blk.k_norms, blk.ve_gates, blk.attn_gates):
            a = an(x)
            vgo = vg(a[..., :32]) if isinstance(vg, nn.Linear) else None
            x = x + attn(a, ve, cos_sin, self.window_sizes[i], qn, kn, vgo, ag(a[..., :12]))
        x = x + mlp(blk.mlp_norm(x))
        if self.training and blk.drop_prob > 0:
            keep = (torch.rand((), device=x.device) >= blk.drop_prob).to(x.dtype)
            x = x_in + keep * (x - x_in)
        return x

    def forward(self, idx, targets=None, loss_reduction="mean"):
        c = self.config
        T = idx.size(1)
        cos_sin = (self.rotary.cos[:, :T].to(torch.float32), self.rotary.sin[:, :T].to(torch.float32))
        x = F.rms_norm(self.transformer.wte(idx), (c.n_embd,))
        x0 = x
        enc = []
        for i in range(self.active_encoder_layers):
            x = self._run_layer(x, x0, cos_sin, i, self.encoder_attns, self.encoder_mlp)
            enc.append(x)
        for i in range(self.active_decoder_start, self.max_n_layer):
            j = self.max_n_layer - 1 - i
            if 0 <= j < len(enc):
                x = x + self.skip_weights[i - self.max_encoder_layers] * enc[j]
            x = self._run_layer(x, x0, cos_sin, i, self.decoder_attns, self.decoder_mlp)
        x = F.rms_norm(x, (c.n_embd,))
        logits = self.lm_head(x)[..., :c.vocab_size].float()
        if c.logit_cap > 0:
            logits = c.logit_cap * torch.tanh(logits / c.logit_cap)
        if targets is None:
            return logits
        return F.cross_entropy(logits.view(-1, logits.size(-1)), targets.reshape(-1), ignore_index=-1, reduction=loss_reduction)


# =============================================================================== gated delta net attention
def gated_delta_rule(q, k, v, alpha, beta):
    """Recurrent statement of the gated delta rule. q, k: (B, T, H, Dk) (k L2-normalised by the caller), v: (B, T, H, Dv),
    alpha, beta: (B, T, H) with alpha in (0, 1] the decay and beta in (0, 1) the write strength.
        S_t = alpha_t * S_{t-1} (I - beta_t k_t k_t^T) + beta_t v_t k_t^T ;  o_t = S_t q_t
    Returns o: (B, T, H, Dv). O(T Dk Dv) time, state kept in fp32."""
    B, T, H, Dk = q.shape
    Dv = v.size(-1)
    S = torch.zeros(B, H, Dv, Dk, dtype=torch.float32, device=q.device)
    out = []
    qf, kf, vf = q.float(), k.float(), v.float()
    for t in range(T):
        kt, vt, qt = kf[:, t], vf[:, t], qf[:, t]
        a, b = alpha[:, t].float()[..., None, None], beta[:, t].float()[..., None, None]
        Sk = torch.einsum("bhvk,bhk->bhv", S, kt)                       # S k_t
        S = a * (S - b * Sk.unsqueeze(-1) * kt.unsqueeze(-2)) + b * vt.unsqueeze(-1) * kt.unsqueeze(-2)
        out.append(torch.einsum("bhvk,bhk->bhv", S, qt))
    return torch.stack(out, dim=1).to(v.dtype)


class GatedDeltaNetAttention(nn.Module):
    """Drop-in replacement for softmax attention on selected layers of the hybrid model: projections, optional
    depth-wise causal convolutions (kernel 4) on q/k/v, SiLU, L2-normalised q/k, data-dependent decay and write
    gates, gated RMSNorm on the output."""

    def __init__(self, n_embd: int, n_head: int, head_dim: Optional[int] = None, use_conv: bool = True, conv_size: int = 4):
        super().__init__()
        self.n_head = n_head
        self.head_dim = head_dim or n_embd // n_head
        inner = self.n_head * self.head_dim
        self.c_q, self.c_k, self.c_v = (nn.Linear(n_embd, inner, bias=False) for _ in range(3))
        self.a_proj = nn.Linear(n_embd, n_head, bias=False)      # decay logits
        self.b_proj = nn.Linear(n_embd, n_head, bias=False)      # write-strength logits
        self.g_proj = nn.Linear(n_embd, inner, bias=False)       # output gate
        self.c_proj = nn.Linear(inner, n_embd, bias=False)
        self.A_log = nn.Parameter(torch.zeros(n_head))
        self.dt_bias = nn.Parameter(torch.zeros(n_head))
        self.use_conv = use_conv
        if use_conv:
            self.convs = nn.ModuleList([nn.Conv1d(inner, inner, conv_size, groups=inner, padding=conv_size - 1, bias=False)
                                        for _ in range(3)])

    def _conv(self, x, conv):
        T = x.size(1)
        return conv(x.transpose(1, 2))[..., :T].transpose(1, 2)

    def forward(self, x):
        B, T, _ = x.shape
        H, D = self.n_head, self.head_dim
        q, k, v = self.c_q(x), self.c_k(x), self.c_v(x)
        if self.use_conv:
            q, k, v = (self._conv(t, c) for t, c in zip((q, k, v), self.convs))
        q, k, v = (F.silu(t).view(B, T, H, D) for t in (q, k, v))
        q = F.normalize(q.float(), dim=-1).to(x.dtype) * D ** -0.5
        k = F.normalize(k.float(), dim=-1).to(x.dtype)
        alpha = torch.exp(-torch.exp(self.A_log.float()) * F.softplus(self.a_proj(x).float() + self.dt_bias.float()))
        beta = torch.sigmoid(self.b_proj(x).float())
        o = gated_delta_rule(q, k, v, alpha, beta)
        o = F.rms_norm(o, (D,)) * F.silu(self.g_proj(x).view(B, T, H, D))
        return self.c_proj(o.reshape(B, T, H * D))
