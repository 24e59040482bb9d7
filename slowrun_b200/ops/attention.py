"""CUDA attention back ends behind `ops.functional.attention`.

`install_default_attention()` picks, in order: the in-tree sm_100a flash-attention kernels when they are built and
enabled, else the flash-attn 2 wheel of the image, else torch SDPA. The last two are library kernels — the same
ones the reference ends up on when run on a B200 (its FlashAttention-3 binary is Hopper-only, train.py:192-207;
its own fallback is SDPA with a dense mask, tiny/train.py:349-365).
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from . import functional as ops

_state = {"name": None}


def _sdpa(q, k, v, window, scale):
    return ops.attention_ref(q, k, v, window, scale)


def _make_fa2():
    from flash_attn import flash_attn_func

    def fa2(q, k, v, window, scale):
        T = q.size(1)
        ws = (-1, -1) if (window is None or window < 0 or window >= T) else (int(window), 0)
        return flash_attn_func(q, k, v, causal=True, window_size=ws, softmax_scale=scale)
    # probe once: the wheel may not carry code for this GPU
    x = torch.randn(1, 128, 1, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    fa2(x, x, x, 64, None).sum().backward()
    torch.cuda.synchronize()
    return fa2


def install_default_attention(prefer: str | None = None) -> str:
    """Chooses the CUDA attention implementation; returns its name ('native', 'flash_attn2' or 'sdpa')."""
    prefer = prefer or os.environ.get("SLOWRUN_ATTN", "auto")
    if not torch.cuda.is_available():
        _state["name"] = "sdpa"
        return "sdpa"
    if prefer in ("auto", "native"):
        try:
            from .flash_attention import native_attention, native_available
            if native_available():
                ops.set_attention_impl(native_attention)
                _state["name"] = "native"
                return "native"
        except ImportError:
            pass
        if prefer == "native":
            raise RuntimeError("native attention kernels requested but not available")
    if prefer in ("auto", "flash_attn2"):
        try:
            ops.set_attention_impl(_make_fa2())
            _state["name"] = "flash_attn2"
            return "flash_attn2"
        except Exception:  # noqa: BLE001
            if prefer == "flash_attn2":
                raise
    ops.set_attention_impl(_sdpa)
    _state["name"] = "sdpa"
    return "sdpa"


def current_attention() -> str | None:
    return _state["name"]
