"""Research model variants of the reference repository, as plain-PyTorch modules (autograd, any device):

* `UniversalGPT` — the universal-transformer fork (research/universal_transformer/train.py:221-330, 432-437,
  530-584): each half of the U-Net shares TWO attention modules and ONE SwiGLU MLP (hidden 8d) across all of its
  layers; what is per-layer are learnable RMSNorms (weight + bias) for the attention inputs, q, k and the MLP input,
  the value / attention gates, lambdas and value projections. The number of active layers grows during training
  (`--depth-schedule "0:10,1533:20"`), new layers being inserted towards the middle of the U-Net.
  The unlimited variant (research/universal_transformer/train_unlimited.py:367-369, 598-604) adds a separate
  `mtp_head` that predicts the token after next from the same final hidden state.

The hybrid softmax / linear-attention fork lives in `models/hybrid.py`. These models run on plain PyTorch ops
(bf16 autocast on a GPU) and on the package's sharded Muon/AdamW optimizer; they are capability surface, not the
tuned flagship.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as ops
from .gpt import ArenaModelMixin, Rotary, has_ve


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
    use_iha: bool = True
    iha_mix_v: bool = True
    mtp_weight: float = 0.0          # > 0: separate mtp_head on the final hidden state (the unlimited variant)
    # switches the shared parameter-grouping code reads
    attn_gate_adamw: bool = False
    xsa_mode: str = "off"


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

    adamw_kind = "norm"

    def adamw_scalar_params(self):
        """Stepped by AdamW at the scalar rate, not by Muon (research/universal_transformer/train.py:487-511)."""
        return [self.weight, self.bias]

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
        self.use_iha, self.iha_mix_v = c.use_iha, c.iha_mix_v
        if self.use_iha:          # head mixing of the projection weights, as in the limited track (train.py:266-298)
            self.q_mix = nn.Parameter(torch.eye(self.n_head))
            self.k_mix = nn.Parameter(torch.eye(self.n_head))
            if self.iha_mix_v:
                self.v_mix = nn.Parameter(torch.eye(self.n_head))

    def _proj(self, x, lin, mix):
        w = lin.weight
        if mix is not None:
            w = (mix @ w.view(self.n_head, -1)).view_as(w)
        return F.linear(x, w.to(x.dtype))

    def forward(self, x, ve, cos_sin, window, q_norm, k_norm, ve_gate, attn_gate):
        B, T, _ = x.shape
        H, D = self.n_head, self.head_dim
        q = self._proj(x, self.c_q, self.q_mix if self.use_iha else None).view(B, T, H, D)
        k = self._proj(x, self.c_k, self.k_mix if self.use_iha else None).view(B, T, H, D)
        v = self._proj(x, self.c_v, self.v_mix if (self.use_iha and self.iha_mix_v) else None).view(B, T, H, D)
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


class UniversalGPT(ArenaModelMixin, nn.Module):
    wire_fused = False            # forward runs on plain PyTorch ops; the arena only serves the optimizer

    def __init__(self, c: UniversalConfig):
        super().__init__()
        self.config = c
        self.arena = None
        self.mtp_weight = c.mtp_weight
        L = c.n_layer
        assert L % 2 == 0
        pv = ((c.vocab_size + 63) // 64) * 64
        self.transformer = nn.ModuleDict({"wte": nn.Embedding(pv, c.n_embd),
                                          "h": nn.ModuleList([LayerParams(c, i) for i in range(L)])})
        self.encoder_attns = nn.ModuleList([SharedAttention(c) for _ in range(2)])
        self.decoder_attns = nn.ModuleList([SharedAttention(c) for _ in range(2)])
        self.encoder_mlp, self.decoder_mlp = SharedMLP(c), SharedMLP(c)
        self.lm_head = nn.Linear(c.n_embd, pv, bias=False)
        if c.mtp_weight > 0:
            self.mtp_head = nn.Linear(c.n_embd, pv, bias=False)
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
        if c.mtp_weight > 0:
            nn.init.normal_(self.mtp_head.weight, std=0.001)
        for m in list(self.encoder_attns) + list(self.decoder_attns):
            for lin in (m.c_q, m.c_k, m.c_v):
                nn.init.uniform_(lin.weight, -s, s)
            nn.init.zeros_(m.c_proj.weight)
            if m.use_iha:
                for mix in (m.q_mix, m.k_mix) + ((m.v_mix,) if m.iha_mix_v else ()):
                    nn.init.eye_(mix)
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
            for nrm in list(blk.attn_norms) + [blk.mlp_norm] + list(blk.q_norms) + list(blk.k_norms):
                nn.init.ones_(nrm.weight)
                nn.init.zeros_(nrm.bias)
        self.resid_lambdas.fill_(1.0)
        self.x0_lambdas.fill_(0.1)
        self.skip_weights.fill_(1.0)
        self.rotary.reset()

    # ------------------------------------------------------------------ what the shared optimizer code asks of a model
    def all_blocks(self):
        return []

    def iha_params(self):
        out = []
        for m in list(self.encoder_attns) + list(self.decoder_attns):
            if m.use_iha:
                out += [m.q_mix, m.k_mix] + ([m.v_mix] if m.iha_mix_v else [])
        return out

    def muon_matrix_params(self):
        """Shared projections and MLPs, per-layer gate linears, value projections
        (research/universal_transformer/train.py:470-503)."""
        iha = {id(p) for p in self.iha_params()}
        shared = [p for mod in (self.encoder_attns, self.decoder_attns, self.encoder_mlp, self.decoder_mlp)
                  for p in mod.parameters() if id(p) not in iha]
        per_layer = []
        for blk in self.transformer.h:
            per_layer += [g.weight for g in blk.attn_gates]
            per_layer += [g.weight for g in blk.ve_gates if isinstance(g, nn.Linear)]
        return shared + per_layer + list(self.ve_projs.parameters())

    def layer_parameters(self, i):
        """Parameters that only layer i touches (norms, gates, its value projection): what goes idle while the layer is
        not part of the active depth."""
        ps = list(self.transformer.h[i].parameters())
        if str(i) in self.ve_projs:
            ps += list(self.ve_projs[str(i)].parameters())
        return ps

    def inactive_parameters(self):
        idle = [i for i in range(self.max_n_layer) if self.active_encoder_layers <= i < self.active_decoder_start]
        return [p for i in idle for p in self.layer_parameters(i)]

    def estimate_flops(self):
        """6 FLOPs per matmul parameter per use (shared modules count once per active layer) plus attention."""
        c = self.config
        per_layer_shared = sum(p.numel() for p in self.encoder_attns.parameters()) + sum(p.numel() for p in self.encoder_mlp.parameters())
        active = list(range(self.active_encoder_layers)) + list(range(self.active_decoder_start, self.max_n_layer))
        own = sum(p.numel() for i in active for p in self.layer_parameters(i))
        heads = self.lm_head.weight.numel() + (self.mtp_head.weight.numel() if c.mtp_weight > 0 else 0)
        D, T = c.n_embd // c.n_head, c.sequence_len
        attn = sum(2 * 12 * c.n_head * D * min(self.window_sizes[i][0], T) for i in active)     # two attention modules per layer
        return 6 * (len(active) * per_layer_shared + own + heads) + attn

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

        def capped(head, h):
            z = F.linear(h, head.weight.to(h.dtype))[..., :c.vocab_size].float()
            return c.logit_cap * torch.tanh(z / c.logit_cap) if c.logit_cap > 0 else z
        logits = capped(self.lm_head, x)
        if targets is None:
            return logits
        lm_loss = F.cross_entropy(logits.view(-1, logits.size(-1)), targets.reshape(-1), ignore_index=-1, reduction=loss_reduction)
        if loss_reduction != "mean" or c.mtp_weight <= 0:
            return lm_loss
        mtp_logits = capped(self.mtp_head, x[:, :-1])
        mtp_loss = F.cross_entropy(mtp_logits.reshape(-1, mtp_logits.size(-1)), targets[:, 1:].reshape(-1), ignore_index=-1)
        return lm_loss + c.mtp_weight * mtp_loss
