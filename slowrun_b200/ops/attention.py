"""CUDA attention back ends.

An implementation is an object with
    fwd(q, k, v, window, scale) -> (y, saved)      q, k, v, y: contiguous (B, T, H, D) bf16
    bwd(saved, dy) -> (dq, dk, dv)
so the block-level backward (`ops/block.py`) can call it without an autograd graph; `as_autograd()` wraps the same
object for the op-by-op path. `install_default_attention()` picks, in order: the in-tree sm_100a flash-attention
kernels when built, else the flash-attn 2 wheel of the image, else torch SDPA. The last two are library kernels —
the same ones the reference ends up on when run on a B200 (its FlashAttention-3 binary is Hopper-only,
train.py:192-207; its own fallback is SDPA with a dense mask, tiny/train.py:349-365). Keys visible to query i are
[i - window, i] (flash-attn's `window_size=(window, 0)` with causal=True).
"""
from __future__ import annotations

import os

import torch

from . import functional as ops

_state = {"impl": None}


class SDPAAttention:
    name = "sdpa"

    def fwd(self, q, k, v, window, scale):
        with torch.enable_grad():
            ql, kl, vl = (t.detach().requires_grad_(True) for t in (q, k, v))
            y = ops.attention_ref(ql, kl, vl, window, scale)
        return y.detach(), (ql, kl, vl, y)

    def bwd(self, saved, dy):
        ql, kl, vl, y = saved
        return torch.autograd.grad(y, (ql, kl, vl), dy)


class FlashAttn2:
    name = "flash_attn2"

    def __init__(self):
        from flash_attn import flash_attn_interface as fai
        self._f = fai._wrapped_flash_attn_forward
        self._b = fai._wrapped_flash_attn_backward
        x = torch.randn(1, 128, 1, 128, device="cuda", dtype=torch.bfloat16)   # probe: the wheel may lack this arch
        y, s = self.fwd(x, x, x, 64, None)
        self.bwd(s, y)
        torch.cuda.synchronize()

    @staticmethod
    def _win(window, T):
        return (-1, -1) if (window is None or window < 0 or window >= T) else (int(window), 0)

    def fwd(self, q, k, v, window, scale):
        wl, wr = self._win(window, q.size(1))
        sc = float(scale) if scale is not None else q.size(-1) ** -0.5
        out, lse, _, rng = self._f(q, k, v, 0.0, sc, True, wl, wr, 0.0, None, False)
        return out, (q, k, v, out, lse, rng, sc, wl, wr)

    def bwd(self, saved, dy):
        q, k, v, out, lse, rng, sc, wl, wr = saved
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        self._b(dy.contiguous(), q, k, v, out, lse, dq, dk, dv, 0.0, sc, True, wl, wr, 0.0, None, False, rng)
        return dq, dk, dv


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, impl, window, scale):
        y, saved = impl.fwd(q.contiguous(), k.contiguous(), v.contiguous(), window, scale)
        ctx.impl, ctx.saved = impl, saved
        return y

    @staticmethod
    def backward(ctx, dy):
        dq, dk, dv = ctx.impl.bwd(ctx.saved, dy)
        return dq, dk, dv, None, None, None


def as_autograd(impl):
    def fn(q, k, v, window, scale):
        return _AttnFn.apply(q, k, v, impl, window, scale)
    return fn


def install_default_attention(prefer: str | None = None) -> str:
    """Chooses the CUDA attention implementation; returns its name ('native', 'flash_attn2' or 'sdpa')."""
    prefer = prefer or os.environ.get("SLOWRUN_ATTN", "auto")
    impl = None
    if torch.cuda.is_available():
        if prefer in ("auto", "native"):
            try:
                from .flash_attention import NativeAttention, native_available
                if native_available():
                    impl = NativeAttention()
            except ImportError:
                impl = None
            if impl is None and prefer == "native":
                raise RuntimeError("native attention kernels requested but not available")
        if impl is None and prefer in ("auto", "flash_attn2"):
            try:
                impl = FlashAttn2()
            except Exception:  # noqa: BLE001
                if prefer == "flash_attn2":
                    raise
    if impl is None:
        impl = SDPAAttention()
    _state["impl"] = impl
    ops.set_attention_impl(as_autograd(impl))
    return impl.name


def current_impl():
    if _state["impl"] is None:
        install_default_attention()
    return _state["impl"]


def current_attention() -> str | None:
    return None if _state["impl"] is None else _state["impl"].name
