"""The Slowrun GPT family as one module with feature switches.

Parameter names, shapes and registration order match the reference modules, so a `{name: tensor}` checkpoint
moves between the two unchanged (limited: train.py:248-383, tiny: tiny/train.py:410-525, two-hour adds the YaRN
rotary tables: two_hour/train.py:291-331). What differs is the execution: eager ops from `slowrun_b200.ops` with
hand-written backward, bf16 shadow weights kept in fused layouts ([c_q;c_k;c_v] and [c_gate;c_fc] feed one GEMM
each), fp32 gradient accumulation inside the weight-gradient GEMM epilogue, and no torch.compile.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import ModelConfig
from ..ops import functional as ops
from ..ops.gemm import gemm
from ..ops import _lib
from ..ops.block import block_forward, block_supported


def has_ve(layer_idx: int, n_layer: int) -> bool:
    """Value projections on alternating layers, last layer always included (train.py:238-240)."""
    return layer_idx % 2 == (n_layer - 1) % 2


class Rotary(nn.Module):
    """Rotary position tables, bf16 [1, T, 1, D/2], for the three RoPE flavours of the model family:
    full (train.py:424-430), half-truncated where only the first D/4 frequency pairs rotate (tiny/train.py:557-567),
    and YaRN-rescalable together with the attention softmax scale (two_hour/train.py:291-331).

    State is the per-pair angular frequency vector `inv_freq`; the tables are a pure function of it
    (`_tabulate`). Stretching the context from L to L' multiplies each frequency by
    s + w (1 - s), s = L / L', where w ramps from 0 to 1 as the number of full turns the pair makes over L goes from
    `slow` to `fast` (slowly rotating pairs are interpolated, fast ones kept), and the softmax scale by 0.2 ln(L'/L) + 1.
    """

    def __init__(self, head_dim: int, max_seq_len: int, base: float = 10000.0, truncate: bool = False):
        super().__init__()
        self.head_dim, self.max_seq_len, self.base, self.truncate = head_dim, max_seq_len, base, truncate
        pairs = head_dim // 2
        self.register_buffer("inv_freq", torch.empty(pairs), persistent=False)
        self.register_buffer("cos", torch.empty(1, max_seq_len, 1, pairs, dtype=torch.bfloat16), persistent=False)
        self.register_buffer("sin", torch.empty(1, max_seq_len, 1, pairs, dtype=torch.bfloat16), persistent=False)
        self.attn_scale = head_dim ** -0.5
        self.yarn_active = False

    def _base_frequencies(self, device):
        pairs = self.head_dim // 2
        live = pairs // 2 if self.truncate else pairs          # pairs that actually rotate
        k = torch.arange(live, dtype=torch.float32, device=device)
        freq = 1.0 / (self.base ** (k / live))
        return torch.cat([freq, freq.new_zeros(pairs - live)])

    @torch.no_grad()
    def _tabulate(self):
        angle = torch.arange(self.max_seq_len, dtype=torch.float32, device=self.inv_freq.device)[:, None] * self.inv_freq
        self.cos.copy_(angle.cos().bfloat16().view_as(self.cos))
        self.sin.copy_(angle.sin().bfloat16().view_as(self.sin))

    @torch.no_grad()
    def reset(self):
        self.inv_freq.copy_(self._base_frequencies(self.inv_freq.device))
        self._tabulate()
        self.attn_scale = self.head_dim ** -0.5
        self.yarn_active = False

    @torch.no_grad()
    def apply_yarn(self, old_window: int, new_window: int, slow: float = 1.0, fast: float = 32.0):
        if new_window <= old_window:
            raise ValueError(f"the context can only be stretched: {old_window} -> {new_window} tokens is not an expansion")
        shrink = old_window / new_window
        turns = self.inv_freq * (old_window / (2 * math.pi))
        keep = ((turns - slow) / (fast - slow)).clamp_(0, 1)
        self.inv_freq.mul_(shrink + keep * (1 - shrink))
        self._tabulate()
        self.attn_scale *= 0.2 * math.log(new_window / old_window) + 1
        self.yarn_active = True


class CausalSelfAttention(nn.Module):
    def __init__(self, config: ModelConfig, layer_idx: int):
        super().__init__()
        self.n_head, self.n_kv_head, self.n_embd = config.n_head, config.n_kv_head, config.n_embd
        self.head_dim = self.n_embd // self.n_head
        assert self.n_embd % self.n_head == 0
        assert self.n_kv_head == self.n_head, "all reference configurations use n_kv_head == n_head"
        d = self.n_embd
        self.c_q = nn.Linear(d, self.n_head * self.head_dim, bias=False)
        self.c_k = nn.Linear(d, self.n_kv_head * self.head_dim, bias=False)
        self.c_v = nn.Linear(d, self.n_kv_head * self.head_dim, bias=False)
        self.c_proj = nn.Linear(d, d, bias=False)
        self.ve_gate_channels = 32
        self.ve_gate = nn.Linear(self.ve_gate_channels, self.n_kv_head, bias=False) if has_ve(layer_idx, config.n_layer) else None
        self.attn_gate_channels = 12
        self.attn_gate = nn.Linear(self.attn_gate_channels, self.n_head, bias=False)
        self.use_iha = config.use_iha
        self.iha_mix_v = config.iha_mix_v
        if self.use_iha:
            self.q_mix = nn.Parameter(torch.zeros(self.n_head, self.n_head))
            self.k_mix = nn.Parameter(torch.zeros(self.n_kv_head, self.n_kv_head))
            if self.iha_mix_v:
                self.v_mix = nn.Parameter(torch.zeros(self.n_kv_head, self.n_kv_head))
        pattern = config.window_pattern.upper()
        is_long = pattern[layer_idx % len(pattern)] == "L" or layer_idx == config.n_layer - 1
        self.use_key_offset = config.key_offset and is_long
        self.xsa_eps = config.xsa_eps
        self.dropout = config.dropout
        self.fused = None  # set by GPT.finalize(): bf16 shadow / gradient views for the CUDA path


class MLP(nn.Module):
    def __init__(self, config: ModelConfig):
        super().__init__()
        h = config.hidden
        self.c_gate = nn.Linear(config.n_embd, h, bias=False)
        self.c_fc = nn.Linear(config.n_embd, h, bias=False)
        self.c_proj = nn.Linear(h, config.n_embd, bias=False)
        self.dropout = config.dropout if config.mlp_dropout else 0.0
        self.fused = None


class Block(nn.Module):
    def __init__(self, config: ModelConfig, layer_idx: int):
        super().__init__()
        self.attn = CausalSelfAttention(config, layer_idx)
        self.mlp = MLP(config)
        self.drop_prob = config.stoch_depth * (layer_idx / max(config.n_layer - 1, 1))


class _IHAFuse(torch.autograd.Function):
    """W'[p] = mix[p] @ W[p].view(H, D*d) for the stacked projections p (train.py:277-280), on bf16 shadows.
    Backward returns the mix gradients to autograd and accumulates mix^T @ dW' into the fp32 weight gradients."""

    @staticmethod
    def forward(ctx, mixes, w16, grad_acc, H):
        P = mixes.size(0)
        m16 = mixes.to(torch.bfloat16)
        out = torch.bmm(m16, w16.view(P, H, -1))
        ctx.save_for_backward(m16, w16)
        ctx.grad_acc, ctx.H = grad_acc, H
        return out.view(w16.shape)

    @staticmethod
    def backward(ctx, dwp):
        m16, w16 = ctx.saved_tensors
        P, H = m16.size(0), ctx.H
        d3 = dwp.reshape(P, H, -1)
        dmix = torch.bmm(d3, w16.view(P, H, -1).transpose(1, 2)).float()
        dw = torch.bmm(m16.transpose(1, 2), d3)
        acc = ctx.grad_acc
        rc = _lib.fn("sr_acc_bf16_into_f32", [_lib.c_void_p, _lib.c_void_p, _lib.ctypes.c_long, _lib.c_void_p])(
            acc.data_ptr(), dw.data_ptr(), dw.numel(), _lib.stream_ptr())
        _lib.check_rc(rc, "sr_acc_bf16_into_f32")
        return dmix, None, None, None


class ArenaModelMixin:
    """What the sharded optimizer needs from a model: parameters and gradients laid out in stacked arenas."""

    def finalize(self, world_size: int = 1, alloc=None):
        """Move parameters and gradients into stacked arenas (plus bf16 shadows and fused operand views on CUDA)."""
        from ..optim.arena import ParamArena
        self.arena = ParamArena(self, world_size, alloc)
        return self

    def zero_grad_arena(self):
        if self.arena is not None:
            self.arena.zero_grads()
        else:
            for p in self.parameters():
                if p.grad is not None:
                    p.grad.zero_()

    def get_device(self):
        return self.transformer.wte.weight.device


class GPT(ArenaModelMixin, nn.Module):
    def __init__(self, config: ModelConfig, pad_vocab_size_to: int = 64):
        super().__init__()
        self.config = config
        c = config
        self.window_pattern = c.window_pattern.upper()
        self.short_window, self.long_window = c.sequence_len // 2, c.sequence_len
        self.window_sizes = self._compute_window_sizes(self.short_window, self.long_window)
        padded_vocab = ((c.vocab_size + pad_vocab_size_to - 1) // pad_vocab_size_to) * pad_vocab_size_to
        self.padded_vocab = padded_vocab
        self.transformer = nn.ModuleDict({
            "wte": nn.Embedding(padded_vocab, c.n_embd),
            "h": nn.ModuleList([Block(c, i) for i in range(c.n_layer)]),
        })
        if c.lm_head_transposed:
            self.lm_head = nn.Module()
            self.lm_head.weight = nn.Parameter(torch.empty(c.n_embd, padded_vocab, dtype=torch.bfloat16))
        else:
            self.lm_head = nn.Linear(c.n_embd, padded_vocab, bias=False)
        self.resid_lambdas = nn.Parameter(torch.ones(c.n_layer))
        self.x0_lambdas = nn.Parameter(torch.zeros(c.n_layer))
        head_dim = c.head_dim
        kv_dim = c.n_kv_head * head_dim
        self.ve_projs = nn.ModuleDict({str(i): nn.Linear(c.n_embd, kv_dim, bias=False)
                                       for i in range(c.n_layer) if has_ve(i, c.n_layer)})
        self.encoder_layers = c.n_layer // 2
        self.skip_weights = nn.Parameter(torch.ones(self.encoder_layers))
        if c.xsa_mode != "off" or c.fused_mtp:
            self.xsa_alphas = nn.Parameter(torch.zeros(c.n_layer, c.n_head))
        self.rotary_seq_len = c.sequence_len * 10
        self.rotary = Rotary(head_dim, self.rotary_seq_len, truncate=c.rope_truncate)
        self._dupe_layers = None
        self._dupe_loops = 0
        self.mtp_weight = c.mtp_weight
        if self.mtp_weight > 0:
            self.mtp_proj = nn.Linear(2 * c.n_embd, c.n_embd, bias=False)
            self.mtp_block = Block(c, c.n_layer)
        self.use_fused_blocks = True   # CUDA: run each block as one autograd node (ops/block.py)
        # Optional callable(layer_index): called during backward once the gradient flowing INTO layer `layer_index`
        # (first time it ran in the forward pass) is complete, i.e. when every weight gradient of that layer and of all
        # later layers has been written. Index n_layer stands for the extra multi-token-prediction block. Used to start
        # gradient reductions while the rest of the backward pass still runs.
        self.layer_done_hook = None
        self._hooked_layers = set()
        self.arena = None          # set by finalize()
        self.norm_eps: Optional[float] = None   # None = torch default for the activation dtype

    # ------------------------------------------------------------------ structure helpers
    def _compute_window_sizes(self, short_w, long_w):
        """(left, right) attention window per layer: the pattern string is tiled over the layers ('S' = short, 'L' =
        long) and the last layer always sees the long window (train.py:432-438)."""
        n, pat = self.config.n_layer, self.window_pattern
        return [((long_w if (pat[i % len(pat)] == "L" or i == n - 1) else short_w), 0) for i in range(n)]

    @torch.no_grad()
    def set_window_sizes(self, short_window: int, long_window: int, apply_yarn: bool = False):
        """Switch the active attention windows (the two-hour track's window schedule, two_hour/train.py:538-551).
        With `apply_yarn` a longer long window also rescales the rotary frequencies and the softmax scale; the long
        window never shrinks once YaRN is in play, because the frequency rescaling is not undone."""
        short_window, long_window = int(short_window), int(long_window)
        if not 0 < short_window <= long_window <= self.config.sequence_len:
            raise ValueError(f"windows must satisfy 0 < short <= long <= {self.config.sequence_len}, "
                             f"got short={short_window}, long={long_window}")
        if apply_yarn and long_window < self.long_window:
            raise ValueError(f"the long window cannot shrink under YaRN: {self.long_window} -> {long_window}")
        if apply_yarn and long_window > self.long_window:
            self.rotary.apply_yarn(self.long_window, long_window)
        self.short_window, self.long_window = short_window, long_window
        self.window_sizes = self._compute_window_sizes(short_window, long_window)

    def set_dupe_layers(self, start: int, end: int, loops: int = 2):
        """Replay decoder layers [start, end) `loops` extra times per forward (train.py:378-383). Only decoder layers
        can be replayed: every replay re-adds the U-Net skip of the matching encoder layer."""
        if not self.encoder_layers <= start < end <= self.config.n_layer:
            raise ValueError(f"replayed layers [{start}, {end}) must lie in the decoder half "
                             f"[{self.encoder_layers}, {self.config.n_layer})")
        self._dupe_layers = (start, end)
        self._dupe_loops = loops

    def clear_dupe_layers(self):
        self._dupe_layers = None

    def all_blocks(self):
        blocks = list(self.transformer.h)
        if self.mtp_weight > 0:
            blocks.append(self.mtp_block)
        return blocks

    def _xsa_enabled(self, i):
        m = self.config.xsa_mode
        if m == "off":
            return False
        if m == "first6":
            return i < min(6, self.config.n_layer)
        if m == "all":
            return True
        raise ValueError(f"unknown xsa_mode: {m}")

    # ------------------------------------------------------------------ init (train.py:385-422, tiny/train.py:527-555)
    @torch.no_grad()
    def init_weights(self):
        c = self.config
        torch.nn.init.normal_(self.transformer.wte.weight, mean=0.0, std=1.0)
        torch.nn.init.normal_(self.lm_head.weight, mean=0.0, std=0.001)
        s = 3 ** 0.5 * c.n_embd ** -0.5
        normal_std = c.n_embd ** -0.5
        if self.mtp_weight > 0:
            torch.nn.init.uniform_(self.mtp_proj.weight, -s, s)
        for block in self.all_blocks():
            if getattr(block.attn, "is_linear_attention", False):
                block.attn.reset_parameters(s)            # token mixers of the hybrid fork bring their own initialisation
            else:
                torch.nn.init.uniform_(block.attn.c_q.weight, -s, s)
                torch.nn.init.uniform_(block.attn.c_k.weight, -s, s)
                torch.nn.init.uniform_(block.attn.c_v.weight, -s, s)
                if c.cproj_zero_init:
                    torch.nn.init.zeros_(block.attn.c_proj.weight)
                else:
                    torch.nn.init.normal_(block.attn.c_proj.weight, mean=0.0, std=normal_std)
            torch.nn.init.uniform_(block.mlp.c_gate.weight, -s, s)
            torch.nn.init.uniform_(block.mlp.c_fc.weight, -s, s)
            if c.cproj_zero_init:
                torch.nn.init.zeros_(block.mlp.c_proj.weight)
            else:
                torch.nn.init.normal_(block.mlp.c_proj.weight, mean=0.0, std=normal_std)
            if not c.cproj_zero_init:   # limited order: gates and mixes inside the block loop
                self._init_gates(block)
        self.resid_lambdas.fill_(c.resid_lambda_init)
        self.x0_lambdas.fill_(0.1)
        if hasattr(self, "xsa_alphas"):
            self.xsa_alphas.zero_()
        for proj in self.ve_projs.values():
            torch.nn.init.uniform_(proj.weight, -s, s)
        if c.cproj_zero_init:
            for block in self.all_blocks():
                self._init_gates(block)
        self.skip_weights.fill_(1.0)
        self.rotary.reset()
        if self.transformer.wte.weight.device.type == "cuda":
            self.transformer.wte.to(dtype=torch.bfloat16)

    @staticmethod
    def _init_gates(block):
        if getattr(block.attn, "is_linear_attention", False):
            return
        if block.attn.ve_gate is not None:
            torch.nn.init.zeros_(block.attn.ve_gate.weight)
        torch.nn.init.zeros_(block.attn.attn_gate.weight)
        if block.attn.use_iha:
            torch.nn.init.eye_(block.attn.q_mix)
            torch.nn.init.eye_(block.attn.k_mix)
            if block.attn.iha_mix_v:
                torch.nn.init.eye_(block.attn.v_mix)

    # ------------------------------------------------------------------ FLOPs per token
    @staticmethod
    def _mean_visible_keys(window: int, T: int) -> float:
        """Average, over the T query positions of a sequence, of the number of keys a causal query with left window
        `window` attends to: position i sees min(i, window) + 1 keys."""
        if window < 0 or window >= T - 1:
            return (T + 1) / 2
        w = min(window + 1, T)
        return w - w * (w - 1) / (2 * T)          # the first w positions see 1..w keys, the other T - w see w

    def estimate_flops(self, num_iterations: Optional[int] = None):
        """Training FLOPs per token in the reference's accounting (train.py:443-459; recurrent form
        tiny/train.py:595-625): 6 per matmul parameter (embedding table and per-layer scalars excluded) plus
        12 * heads * head_dim * mean visible keys per layer for attention. For the recurrent (tiny) model the layer
        stack and the value projections count once per pass."""
        c = self.config
        total = sum(p.numel() for p in self.parameters())
        scalars = [self.resid_lambdas, self.x0_lambdas, self.skip_weights] + ([self.xsa_alphas] if hasattr(self, "xsa_alphas") else [])
        dense = total - self.transformer.wte.weight.numel() - sum(p.numel() for p in scalars)
        attn = sum(12 * c.n_head * c.head_dim * self._mean_visible_keys(w[0], c.sequence_len) for w in self.window_sizes)
        recurrent = c.num_iterations > 1 or num_iterations is not None
        if not recurrent:
            return 6 * dense + attn
        passes = c.num_iterations if num_iterations is None else num_iterations
        per_pass = sum(p.numel() for p in self.transformer.h.parameters()) + sum(p.numel() for p in self.ve_projs.parameters())
        return 6 * (dense - per_pass + passes * per_pass) + passes * attn

    # ------------------------------------------------------------------ block forward
    def _eps(self, x):
        return self.norm_eps

    def _attn_forward(self, attn: CausalSelfAttention, a, ve, cos_sin, window, scale, xsa_alpha):
        B, T, C = a.shape
        H, D = attn.n_head, attn.head_dim
        cuda = a.is_cuda
        fz = attn.fused
        if cuda:
            if attn.use_iha:
                mixes = torch.stack([attn.q_mix, attn.k_mix, attn.v_mix]) if attn.iha_mix_v else \
                    torch.stack([attn.q_mix, attn.k_mix, torch.eye(H, device=a.device, dtype=attn.q_mix.dtype)])
                w_qkv = _IHAFuse.apply(mixes, fz["qkv_w16"].view(3, H * D, C), fz["qkv_grad"].view(3, H * D, C), H).view(3 * H * D, C)
                qkv = ops.linear(a, w_qkv)
            else:
                qkv = ops.linear(a, fz["qkv_w16"], fz["qkv_grad"])
            qkv = qkv.view(B, T, 3, H, D)
            q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        else:
            def proj(lin, mix):
                w = lin.weight
                if mix is not None:
                    w = (mix @ w.view(H, D, -1).flatten(1)).view_as(w)
                return F.linear(a, w.to(a.dtype)).view(B, T, H, D)
            q = proj(attn.c_q, attn.q_mix if attn.use_iha else None)
            k = proj(attn.c_k, attn.k_mix if attn.use_iha else None)
            v = proj(attn.c_v, attn.v_mix if (attn.use_iha and attn.iha_mix_v) else None)
        if ve is not None:
            gate = 2 * torch.sigmoid(F.linear(a[..., :attn.ve_gate_channels], attn.ve_gate.weight.to(a.dtype)))
            v = ops.gated_add(v, gate, ve.view(B, T, H, D))
        cos, sin = cos_sin
        q = ops.rope_qknorm(q, cos, sin, self.norm_eps)
        k = ops.rope_qknorm(k, cos, sin, self.norm_eps)
        if attn.use_key_offset and T > 1:
            k = torch.cat([k[..., :D // 2], torch.cat([k[:, :1, :, D // 2:], k[:, :-1, :, D // 2:]], dim=1)], dim=-1)
        y = ops.attention(q, k, v, window[0], scale)
        if xsa_alpha is not None:
            alpha = torch.tanh(xsa_alpha).to(y.dtype).view(1, 1, H, 1)
            v_hat = v / v.square().sum(dim=-1, keepdim=True).sqrt().clamp_min(attn.xsa_eps)
            coeff = (y * v_hat).sum(dim=-1, keepdim=True) * alpha
            y = torch.addcmul(y, v_hat, coeff, value=-1.0)
        agate = torch.sigmoid(F.linear(a[..., :attn.attn_gate_channels], attn.attn_gate.weight.to(a.dtype)))
        y = ops.head_scale(y, agate)
        y = y.reshape(B, T, H * D)
        if cuda:
            return ops.linear(y, fz["proj_w16"], fz["proj_grad"])
        return F.linear(y, attn.c_proj.weight.to(y.dtype))

    def _mlp_forward(self, mlp: MLP, n):
        if n.is_cuda:
            fz = mlp.fused
            gf = ops.linear(n, fz["gf_w16"], fz["gf_grad"])
            return ops.linear(ops.swiglu(gf), fz["proj_w16"], fz["proj_grad"])
        g = F.linear(n, mlp.c_gate.weight.to(n.dtype))
        f = F.linear(n, mlp.c_fc.weight.to(n.dtype))
        return F.linear(F.silu(g) * f, mlp.c_proj.weight.to(n.dtype))

    def _block_forward(self, block: Block, x, ve, cos_sin, window, scale, xsa_alpha=None):
        training = self.training
        sd = training and block.drop_prob > 0
        x_in = x
        a = ops.rms_norm(x, self.norm_eps)
        if getattr(block.attn, "is_linear_attention", False):
            attn_out = block.attn(a)
        else:
            attn_out = self._attn_forward(block.attn, a, ve, cos_sin, window, scale, xsa_alpha)
        x = ops.dropout_add(x, attn_out, block.attn.dropout, training)
        n = ops.rms_norm(x, self.norm_eps)
        mlp_out = self._mlp_forward(block.mlp, n)
        if sd:
            keep = (torch.rand((), device=x.device) >= block.drop_prob).float()
            return ops.dropout_add(x, mlp_out, block.mlp.dropout, training, x_in=x_in, keep=keep)
        return ops.dropout_add(x, mlp_out, block.mlp.dropout, training)

    def _ve(self, i, x0):
        key = str(i)
        if key not in self.ve_projs:
            return None
        lin = self.ve_projs[key]
        if x0.is_cuda:
            return ops.linear(x0, lin.fused["w16"], lin.fused["grad"])
        return F.linear(x0, lin.weight.to(x0.dtype))

    def _watch_layer_input(self, i, x):
        hook = self.layer_done_hook
        if hook is not None and i not in self._hooked_layers and torch.is_grad_enabled() and x.requires_grad:
            self._hooked_layers.add(i)
            x.register_hook(lambda g, i=i: hook(i))

    def _layer(self, i, x, x0, skip, cos_sin, scale):
        j = i - self.encoder_layers
        block = self.transformer.h[i]
        self._watch_layer_input(i, x)
        if x.is_cuda and self.use_fused_blocks and block_supported(self, block):
            ve_lin = self.ve_projs[str(i)] if str(i) in self.ve_projs else None
            return block_forward(self, block, x, x0, skip, i, max(j, 0), True, ve_lin, self.window_sizes[i], scale)
        x = ops.lambda_mix(x, x0, skip, self.resid_lambdas, self.x0_lambdas, self.skip_weights, i, max(j, 0))
        ve = self._ve(i, x0)
        xsa = self.xsa_alphas[i] if self._xsa_enabled(i) else None
        return self._block_forward(self.transformer.h[i], x, ve, cos_sin, self.window_sizes[i], scale, xsa)

    def _run_decoder_layers(self, x, x0, enc, start, end, cos_sin, scale):
        n = self.config.n_layer
        for i in range(start, end):
            j = n - 1 - i
            skip = enc[j] if 0 <= j < self.encoder_layers else None
            x = self._layer(i, x, x0, skip, cos_sin, scale)
        return x

    def _run_network_once(self, x, x0, cos_sin, scale):
        """One pass over all layers with U-Net skips and (optionally) replayed decoder layers
        (train.py:533-556; the tiny track pops a skip stack, which pairs layers the same way)."""
        enc = []
        for i in range(self.encoder_layers):
            x = self._layer(i, x, x0, None, cos_sin, scale)
            enc.append(x)
        n = self.config.n_layer
        dupe = self._dupe_layers
        if dupe is None:
            return self._run_decoder_layers(x, x0, enc, self.encoder_layers, n, cos_sin, scale)
        x = self._run_decoder_layers(x, x0, enc, self.encoder_layers, dupe[1], cos_sin, scale)
        for _ in range(self._dupe_loops):
            x = self._run_decoder_layers(x, x0, enc, dupe[0], dupe[1], cos_sin, scale)
        return self._run_decoder_layers(x, x0, enc, dupe[1], n, cos_sin, scale)

    # ------------------------------------------------------------------ heads
    def _head_weight(self):
        """(weight, grad accumulator, transposed?) of the lm head for the op layer."""
        w = self.lm_head.weight
        if not w.is_cuda:
            return w, None, self.config.lm_head_transposed
        if self.config.lm_head_transposed:
            return w, self.arena.head_grad, True
        return self.arena.head_w16, self.arena.head_grad, False

    def _embed(self, idx):
        return ops.rms_norm(self.transformer.wte(idx), self.norm_eps)

    def trunk(self, idx, num_iterations=None):
        """Embedding -> all layers (x num_iterations for the recurrent tiny model) -> final norm."""
        c = self.config
        B, T = idx.size()
        cos_sin = (self.rotary.cos[:, :T], self.rotary.sin[:, :T])
        scale = self.rotary.attn_scale if self.rotary.yarn_active else None
        if self.training and idx.is_cuda:
            ops.advance_dropout_state(idx.device)
        self._hooked_layers = set()
        x = self._embed(idx)
        x_emb = x
        if c.num_iterations > 1 or num_iterations is not None:
            iters = c.num_iterations if num_iterations is None else num_iterations
            if not 1 <= iters <= c.num_iterations + 2:
                raise ValueError(f"num_iterations must be in [1, {c.num_iterations + 2}], got {iters}")
            grad_start = iters - 1 if self.training else 0   # only the last pass is back-propagated
            for it in range(iters):
                if self.training and it < grad_start:
                    with torch.no_grad():
                        x = ops.rms_norm(self._run_network_once(x, x_emb, cos_sin, scale), self.norm_eps)
                    x = x.detach()
                else:
                    x = ops.rms_norm(self._run_network_once(x, x_emb, cos_sin, scale), self.norm_eps)
            return ops.rms_norm(x, self.norm_eps)
        x = self._run_network_once(x, x_emb, cos_sin, scale)
        return ops.rms_norm(x, self.norm_eps)

    def _mtp_loss(self, x, targets, w, acc, w_t):
        """Extra-block multi-token prediction (train.py:569-579): predict targets[t+1] from (x[t], embed(targets[t]))."""
        c = self.config
        mtp_emb = self._embed(targets[:, :-1].clamp(min=0))
        cat = torch.cat([x[:, :-1], mtp_emb], dim=-1)
        if cat.is_cuda:
            combined = ops.linear(cat, self.mtp_proj.fused["w16"], self.mtp_proj.fused["grad"])
        else:
            combined = F.linear(cat, self.mtp_proj.weight.to(cat.dtype))
        self._watch_layer_input(c.n_layer, combined)
        mT = combined.size(1)
        cs = (self.rotary.cos[:, :mT], self.rotary.sin[:, :mT])
        scale = self.rotary.attn_scale if self.rotary.yarn_active else None
        if combined.is_cuda and self.use_fused_blocks and block_supported(self, self.mtp_block):
            mtp_x = block_forward(self, self.mtp_block, combined, None, None, 0, 0, False, None, (-1, -1), scale)
        else:
            mtp_x = self._block_forward(self.mtp_block, combined, None, cs, (-1, -1), scale)
        mtp_out = ops.rms_norm(mtp_x, self.norm_eps)
        return ops.lm_head_loss(mtp_out, w, targets[:, 1:], c.logit_cap, c.vocab_size, acc, w_t)

    def forward(self, idx, targets=None, loss_reduction="mean", num_iterations=None, mtp_weights=None, distill=False,
                label_smoothing=0.0):
        c = self.config
        x = self.trunk(idx, num_iterations)
        w, acc, w_t = self._head_weight()
        if targets is None:
            return ops.lm_head_logits(x, w, c.logit_cap, c.vocab_size, w_t)
        if distill or label_smoothing > 0:
            # unlimited track: logits are needed outside (KL to a teacher) or the loss is label-smoothed
            logits = ops.lm_head_logits_grad(x, w, c.logit_cap, c.vocab_size, acc, w_t)
            mtp_loss = self._mtp_loss(x, targets, w, acc, w_t) if self.mtp_weight > 0 else None
            if distill:
                return logits, mtp_loss
            loss = F.cross_entropy(logits.view(-1, logits.size(-1)), targets.reshape(-1), ignore_index=-1,
                                   label_smoothing=label_smoothing)
            return (loss + self.mtp_weight * mtp_loss if mtp_loss is not None else loss), {"lm_loss": loss}
        if c.fused_mtp and self.training and mtp_weights is not None:
            # tiny: one head scored against shifted targets over the whole padded vocabulary (tiny/train.py:682-696)
            return ops.lm_head_loss(x, w, targets, c.logit_cap, self.padded_vocab, acc, w_t, weights=mtp_weights,
                                    fp8=c.fp8_lm_head)
        if loss_reduction != "mean":
            return ops.lm_head_rows(x, w, targets, c.logit_cap, c.vocab_size, w_t).view(targets.shape)
        lm_loss = ops.lm_head_loss(x, w, targets, c.logit_cap, c.vocab_size, acc, w_t)
        if c.fused_mtp:
            return lm_loss
        if self.mtp_weight <= 0:
            return lm_loss, {"lm_loss": lm_loss}
        mtp_loss = self._mtp_loss(x, targets, w, acc, w_t)
        return lm_loss + self.mtp_weight * mtp_loss, {"lm_loss": lm_loss, "mtp_loss": mtp_loss}


def build_model(config: ModelConfig, device, seed: Optional[int] = 42, world_size: int = 1, alloc=None, factory=None) -> GPT:
    """Construct on `device`, initialise with the reference's RNG call order, and lay out the arenas. `factory(config)`
    builds a GPT subclass instead (the research forks)."""
    device = torch.device(device)
    if seed is not None:
        torch.manual_seed(seed)
        if device.type == "cuda":
            torch.cuda.manual_seed(seed)
    # Built on the meta device and materialised empty, as the reference scripts do (train.py:1044-1047): the module
    # constructors then draw nothing from the generator, so init_weights() starts from the freshly seeded state and
    # the same seed gives the reference's parameters on the GPU as well.
    with torch.device("meta"):
        model = GPT(config) if factory is None else factory(config)
    model.to_empty(device=device)
    model.init_weights()
    if device.type == "cuda":
        model.norm_eps = ops.BF16_EPS
        from ..ops.attention import current_attention, install_default_attention
        if current_attention() is None:
            install_default_attention()
    model.finalize(world_size, alloc)
    return model
