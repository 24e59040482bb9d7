"""In-tree sm_100a flash attention (csrc/flash_attn_fwd.cu, csrc/flash_attn_bwd.cu) behind the attention
implementation interface of `ops/attention.py`. head_dim 128, causal, left sliding window, runtime softmax scale.
The reference gets attention from a prebuilt FlashAttention-3 binary that only exists for Hopper (train.py:192-213).
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib

P, I, L, F32 = _lib.c_void_p, _lib.c_int, ctypes.c_long, _lib.c_float


def _has(symbol: str) -> bool:
    try:
        getattr(_lib.lib(), symbol)
        return True
    except AttributeError:
        return False


def native_available() -> bool:
    if not torch.cuda.is_available() or os.environ.get("SLOWRUN_NATIVE_ATTN", "1") == "0":
        return False
    return _has("sr_flash_attn_fwd")


DEFAULT_BKV = int(os.environ.get("SLOWRUN_ATTN_BKV", "64"))


def native_fwd(q, k, v, window, scale, bkv=None):
    """q, k, v: (B, T, H, 128) bf16, last two dims dense (token stride may be larger). Returns (out, lse[B,H,T])."""
    B, T, H, D = q.shape
    assert D == 128 and q.dtype == torch.bfloat16
    for t in (q, k, v):
        assert t.stride(3) == 1 and t.stride(2) == D and t.stride(0) == T * t.stride(1)
    out = torch.empty((B, T, H, D), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, H, T), dtype=torch.float32, device=q.device)
    w = -1 if (window is None or window < 0 or window >= T) else int(window)
    sc = float(scale) if scale is not None else D ** -0.5
    rc = _lib.fn("sr_flash_attn_fwd", [P] * 5 + [I, I, I, L, L, L, I, F32, I, P, P])(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), B, T, H, q.stride(1), k.stride(1),
        v.stride(1), w, sc, int(bkv or DEFAULT_BKV), _lib.status_buffer(q.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "sr_flash_attn_fwd")
    return out, lse, sc, w


def native_bwd(dout, q, k, v, out, lse, sc, w, delta=None, dq_fp32=False):
    """dq, dk, dv. `delta` (B, H, T) fp32 = rowsum(dout * out) may be supplied by the caller (the head-gate backward
    produces it for free); `dq_fp32` returns dQ as the kernel's fp32 accumulator instead of a bf16 copy."""
    B, T, H, D = q.shape
    dk = torch.empty((B, T, H, D), dtype=torch.bfloat16, device=q.device)
    dv = torch.empty_like(dk)
    dq = None if dq_fp32 else torch.empty_like(dk)
    dq_acc = torch.zeros((B, T, H, D), dtype=torch.float32, device=q.device)
    flags = (1 if delta is not None else 0) | (2 if dq_fp32 else 0)
    if delta is None:
        delta = torch.empty((B, H, T), dtype=torch.float32, device=q.device)
    rc = _lib.fn("sr_flash_attn_bwd_ex", [P] * 11 + [I, I, I, I, F32, I, P, P])(
        dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), delta.data_ptr(),
        dq_acc.data_ptr(), _lib.ptr(dq), dk.data_ptr(), dv.data_ptr(), B, T, H, w, sc, flags,
        _lib.status_buffer(q.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "sr_flash_attn_bwd_ex")
    return (dq_acc if dq_fp32 else dq), dk, dv


class NativeAttention:
    """tcgen05 forward; tcgen05 backward when built, else the flash-attn 2 backward on the same (out, lse)."""

    def __init__(self):
        self.has_bwd = _has("sr_flash_attn_bwd") and os.environ.get("SLOWRUN_NATIVE_ATTN_BWD", "1") != "0"
        self.name = "native" if self.has_bwd else "native_fwd+flash_attn2_bwd"
        self._fa2_bwd = None
        if not self.has_bwd:
            from flash_attn import flash_attn_interface as fai
            self._fa2_bwd = fai._wrapped_flash_attn_backward
        x = torch.randn(1, 256, 1, 128, device="cuda", dtype=torch.bfloat16)   # self-check against SDPA
        y, s = self.fwd(x, x, x, 100, None)
        from .functional import attention_ref
        ref = attention_ref(x.float(), x.float(), x.float(), 100, None)
        torch.cuda.synchronize()
        _lib.check_status()
        if not torch.allclose(y.float(), ref, rtol=3e-2, atol=3e-2):
            raise RuntimeError("native attention self-check failed")

    def fwd(self, q, k, v, window, scale):
        q, k, v = (t if (t.stride(3) == 1 and t.stride(2) == 128) else t.contiguous() for t in (q, k, v))
        out, lse, sc, w = native_fwd(q, k, v, window, scale)
        return out, (q, k, v, out, lse, sc, w)

    def bwd_fused(self, saved, dy, delta):
        """Backward for callers that already hold delta = rowsum(dy * out) and consume dQ in fp32 (the fused block)."""
        q, k, v, out, lse, sc, w = saved
        return native_bwd(dy, q.contiguous(), k.contiguous(), v.contiguous(), out, lse, sc, w, delta=delta, dq_fp32=True)

    def bwd(self, saved, dy):
        q, k, v, out, lse, sc, w = saved
        dy = dy if dy.is_contiguous() else dy.contiguous()
        if self.has_bwd:
            return native_bwd(dy, q.contiguous(), k.contiguous(), v.contiguous(), out, lse, sc, w)
        dq, dk, dv = torch.empty_like(out), torch.empty_like(out), torch.empty_like(out)
        wl, wr = (-1, -1) if w < 0 else (w, 0)
        self._fa2_bwd(dy, q, k, v, out, lse, dq, dk, dv, 0.0, sc, True, wl, wr, 0.0, None, False, None)
        return dq, dk, dv
