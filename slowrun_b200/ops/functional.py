"""Model ops: each has a plain-PyTorch statement (`*_ref`, differentiable, runs anywhere — the CPU path and the
numerics oracle of the GPU tests) and a CUDA path built from the sm_100a kernels with a hand-written backward.

The public functions pick the CUDA path whenever their input lives on a GPU; there is no other backend.
Reference counterparts are cited per op; the reference gets these fused by torch.compile (train.py:1060).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch.autograd import Function

from . import _lib
from .gemm import gemm

c_void_p, c_int, c_long, c_float, c_ull = _lib.c_void_p, _lib.c_int, _lib.ctypes.c_long, _lib.c_float, _lib.ctypes.c_ulonglong

# eps of the weight-less RMSNorm: torch's default for the dtype the reference norms in (bf16 under autocast).
BF16_EPS = float(torch.finfo(torch.bfloat16).eps)


def _eps_for(x: torch.Tensor, eps):
    if eps is not None:
        return float(eps)
    return float(torch.finfo(x.dtype).eps)


def _call(name, argtypes, *args):
    rc = _lib.fn(name, argtypes)(*args)
    _lib.check_rc(rc, name)


def _c(t):
    return t if t.is_contiguous() else t.contiguous()


# =============================================================================== RMSNorm (train.py:235-236)
def rms_norm_ref(x, eps=None):
    return F.rms_norm(x, (x.size(-1),), eps=eps)


class _RMSNormFn(Function):
    @staticmethod
    def forward(ctx, x, eps):
        D = x.size(-1)
        x2 = x.reshape(-1, D)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        y = torch.empty((x2.size(0), D), dtype=torch.bfloat16, device=x.device)
        _call("sr_rmsnorm_fwd", [c_void_p, c_void_p, c_long, c_int, c_long, c_float, c_void_p],
              x2.data_ptr(), y.data_ptr(), x2.size(0), D, x2.stride(0), eps, _lib.stream_ptr())
        ctx.save_for_backward(x2)
        ctx.eps = eps
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        D = x2.size(-1)
        dy2 = _c(dy.reshape(-1, D))
        dx = torch.empty((x2.size(0), D), dtype=torch.bfloat16, device=dy.device)
        _call("sr_rmsnorm_bwd", [c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_long, c_float, c_void_p],
              x2.data_ptr(), dy2.data_ptr(), 0, dx.data_ptr(), x2.size(0), D, x2.stride(0), ctx.eps, _lib.stream_ptr())
        return dx.view(ctx.shape), None


def rms_norm(x, eps=None):
    if x.is_cuda:
        return _RMSNormFn.apply(x, _eps_for(x, eps))
    return rms_norm_ref(x, eps)


# =============================================================================== Linear
def linear_ref(x, w):
    return F.linear(x, w.to(x.dtype))


class _LinearFn(Function):
    """y = x @ w.T on the tcgen05 GEMM. `w` is [N, K] (or [K, N] when w_t) bf16. When `grad_acc` (fp32, same layout
    as w) is given the weight gradient is accumulated into it inside the GEMM epilogue and autograd sees None."""

    @staticmethod
    def forward(ctx, x, w, grad_acc, w_t):
        K = x.size(-1)
        x2 = x.reshape(-1, K)
        if x2.stride(-1) != 1 or (x2.stride(0) % 8) != 0:
            x2 = x2.contiguous()
        y = gemm(x2, w, b_mn=w_t)
        ctx.save_for_backward(x2, w)
        ctx.grad_acc = grad_acc
        ctx.w_t = w_t
        ctx.xshape = x.shape
        N = w.size(1) if w_t else w.size(0)
        return y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        w_t = ctx.w_t
        N = dy.size(-1)
        dy2 = dy.reshape(-1, N)
        if dy2.stride(-1) != 1 or (dy2.stride(0) % 8) != 0 or (dy2.data_ptr() % 16) != 0:
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=not w_t).view(ctx.xshape)
        dw = None
        acc = ctx.grad_acc
        if acc is not None:
            if w_t:   # dW[K, N] = x^T dy
                gemm(x2, dy2, out=acc, cin=acc, a_mn=True, b_mn=True, beta=1.0)
            else:     # dW[N, K] = dy^T x
                gemm(dy2, x2, out=acc, cin=acc, a_mn=True, b_mn=True, beta=1.0)
        elif ctx.needs_input_grad[1]:
            dw = gemm(x2, dy2, a_mn=True, b_mn=True) if w_t else gemm(dy2, x2, a_mn=True, b_mn=True)
        return dx, dw, None, None


def linear(x, w, grad_acc=None, w_t=False):
    """x[..., K] @ W^T with W given as [N, K] (w_t=False) or stored transposed [K, N] (w_t=True)."""
    if x.is_cuda:
        return _LinearFn.apply(x, w, grad_acc, w_t)
    return x @ w.to(x.dtype) if w_t else linear_ref(x, w)


# =============================================================================== lambda mix (train.py:519-522)
def lambda_mix_ref(x, x0, skip, lam_r, lam_0, skip_w):
    if skip is not None:
        x = x + skip_w * skip
    return lam_r * x + lam_0 * x0


class _LambdaMixFn(Function):
    """Scalars are read on the device from the parameter vectors at index (i, j); their gradients are accumulated
    straight into the parameters' fp32 .grad buffers, so autograd sees None for them."""

    @staticmethod
    def forward(ctx, x, x0, skip, resid_l, x0_l, skip_w, i, j):
        x, x0 = _c(x), _c(x0)
        skip = _c(skip) if skip is not None else None
        out = torch.empty_like(x)
        p_lr = resid_l.data_ptr() + 4 * i
        p_l0 = x0_l.data_ptr() + 4 * i
        p_ws = skip_w.data_ptr() + 4 * j if skip is not None else 0
        _call("sr_lambda_mix_fwd", [c_void_p] * 7 + [c_long, c_void_p],
              x.data_ptr(), x0.data_ptr(), _lib.ptr(skip), out.data_ptr(), p_lr, p_l0, p_ws, x.numel(), _lib.stream_ptr())
        ctx.save_for_backward(x, x0, skip if skip is not None else x.new_empty(0), resid_l, x0_l, skip_w)
        ctx.has_skip = skip is not None
        ctx.ij = (i, j)
        return out

    @staticmethod
    def backward(ctx, g):
        x, x0, skip, resid_l, x0_l, skip_w = ctx.saved_tensors
        i, j = ctx.ij
        g = _c(g)
        has_skip = ctx.has_skip
        dx = torch.empty_like(x)
        dx0 = torch.empty_like(x)
        dskip = torch.empty_like(x) if has_skip else None
        dscal = torch.zeros(3, dtype=torch.float32, device=x.device)
        _call("sr_lambda_mix_bwd", [c_void_p] * 11 + [c_long, c_void_p],
              g.data_ptr(), x.data_ptr(), x0.data_ptr(), skip.data_ptr() if has_skip else 0,
              dx.data_ptr(), dx0.data_ptr(), _lib.ptr(dskip),
              resid_l.data_ptr() + 4 * i, x0_l.data_ptr() + 4 * i, skip_w.data_ptr() + 4 * j if has_skip else 0,
              dscal.data_ptr(), x.numel(), _lib.stream_ptr())
        for p, idx, k in ((resid_l, i, 0), (x0_l, i, 1), (skip_w, j, 2)):
            if k == 2 and not has_skip:
                continue
            if p.grad is None:
                p.grad = torch.zeros_like(p)
            p.grad[idx] += dscal[k]
        return dx, dx0, dskip, None, None, None, None, None


def lambda_mix(x, x0, skip, resid_l, x0_l, skip_w, i, j):
    """x_new = resid_l[i] * (x + skip_w[j] * skip) + x0_l[i] * x0  (skip may be None)."""
    if x.is_cuda:
        return _LambdaMixFn.apply(x, x0, skip, resid_l, x0_l, skip_w, i, j)
    return lambda_mix_ref(x, x0, skip, resid_l[i], x0_l[i], skip_w[j] if skip is not None else None)


# =============================================================================== RoPE + QK norm (train.py:242-245, 304-306)
def rope_qknorm_ref(x, cos, sin, eps=None):
    """x: [B, T, H, D]; cos/sin: [1, T, 1, D/2]. Rotation on the half-split layout, then per-head RMSNorm."""
    d = x.shape[3] // 2
    x1, x2 = x[..., :d], x[..., d:]
    cos, sin = cos.to(x.dtype), sin.to(x.dtype)
    y = torch.cat([x1 * cos + x2 * sin, x1 * (-sin) + x2 * cos], 3)
    return F.rms_norm(y, (y.size(-1),), eps=eps)


class _RopeQKNormFn(Function):
    @staticmethod
    def forward(ctx, x, cos, sin, eps):
        B, T, H, D = x.shape
        assert D == 128, "rope_qknorm kernel is written for head_dim 128"
        assert x.stride(3) == 1 and x.stride(2) == D and x.stride(0) == T * x.stride(1)
        out = torch.empty((B, T, H, D), dtype=torch.bfloat16, device=x.device)
        _call("sr_rope_qknorm_fwd", [c_void_p] * 4 + [c_long, c_int, c_int, c_long, c_float, c_void_p],
              x.data_ptr(), out.data_ptr(), cos.data_ptr(), sin.data_ptr(), B * T, H, T, x.stride(1), eps, _lib.stream_ptr())
        ctx.save_for_backward(x, cos, sin)
        ctx.eps = eps
        return out

    @staticmethod
    def backward(ctx, g):
        x, cos, sin = ctx.saved_tensors
        B, T, H, D = x.shape
        g = _c(g)
        dx = torch.empty((B, T, H, D), dtype=torch.bfloat16, device=x.device)
        _call("sr_rope_qknorm_bwd", [c_void_p] * 5 + [c_long, c_int, c_int, c_long, c_long, c_float, c_void_p],
              x.data_ptr(), g.data_ptr(), dx.data_ptr(), cos.data_ptr(), sin.data_ptr(), B * T, H, T, x.stride(1),
              H * D, ctx.eps, _lib.stream_ptr())
        return dx, None, None, None


def rope_qknorm(x, cos, sin, eps=None):
    """x [B,T,H,128] (may be a column slice of a fused projection output) -> contiguous [B,T,H,128]."""
    if x.is_cuda:
        T = x.size(1)
        c2 = _c(cos.reshape(-1, cos.size(-1))[:T])
        s2 = _c(sin.reshape(-1, sin.size(-1))[:T])
        return _RopeQKNormFn.apply(x, c2, s2, _eps_for(x, eps))
    return rope_qknorm_ref(x, cos, sin, eps)


# =============================================================================== per-head gates (train.py:299-303, 308-309)
def gated_add_ref(v, gate, ve):
    return v + gate.unsqueeze(-1).to(v.dtype) * ve


def head_scale_ref(y, gate):
    return y * gate.unsqueeze(-1).to(y.dtype)


def _head_view_ok(t, D):
    return t.stride(3) == 1 and t.stride(2) == D and t.stride(0) == t.size(1) * t.stride(1)


class _GatedAddFn(Function):
    @staticmethod
    def forward(ctx, v, gate, ve):
        B, T, H, D = v.shape
        assert D == 128 and _head_view_ok(v, D) and _head_view_ok(ve, D)
        gate = _c(gate.float())
        out = torch.empty((B, T, H, D), dtype=torch.bfloat16, device=v.device)
        _call("sr_head_gate_fwd", [c_void_p] * 4 + [c_long, c_int, c_long, c_long, c_long, c_int, c_void_p],
              v.data_ptr(), ve.data_ptr(), gate.data_ptr(), out.data_ptr(), B * T, H, v.stride(1), ve.stride(1), H * D, 0,
              _lib.stream_ptr())
        ctx.save_for_backward(gate, ve)
        return out

    @staticmethod
    def backward(ctx, g):
        gate, ve = ctx.saved_tensors
        B, T, H, D = ve.shape
        g = _c(g)
        dve = torch.empty((B, T, H, D), dtype=torch.bfloat16, device=g.device)
        dgate = torch.empty((B, T, H), dtype=torch.float32, device=g.device)
        _call("sr_head_gate_bwd", [c_void_p] * 5 + [c_long, c_int, c_long, c_long, c_long, c_void_p],
              g.data_ptr(), ve.data_ptr(), gate.data_ptr(), dve.data_ptr(), dgate.data_ptr(), B * T, H, H * D,
              ve.stride(1), H * D, _lib.stream_ptr())
        return g, dgate, dve


class _HeadScaleFn(Function):
    @staticmethod
    def forward(ctx, y, gate):
        B, T, H, D = y.shape
        assert D == 128
        y = _c(y)
        gate = _c(gate.float())
        out = torch.empty_like(y)
        _call("sr_head_gate_fwd", [c_void_p] * 4 + [c_long, c_int, c_long, c_long, c_long, c_int, c_void_p],
              y.data_ptr(), 0, gate.data_ptr(), out.data_ptr(), B * T, H, H * D, 0, H * D, 1, _lib.stream_ptr())
        ctx.save_for_backward(y, gate)
        return out

    @staticmethod
    def backward(ctx, g):
        y, gate = ctx.saved_tensors
        B, T, H, D = y.shape
        g = _c(g)
        dy = torch.empty_like(y)
        dgate = torch.empty((B, T, H), dtype=torch.float32, device=g.device)
        _call("sr_head_gate_bwd", [c_void_p] * 5 + [c_long, c_int, c_long, c_long, c_long, c_void_p],
              g.data_ptr(), y.data_ptr(), gate.data_ptr(), dy.data_ptr(), dgate.data_ptr(), B * T, H, H * D, H * D, H * D,
              _lib.stream_ptr())
        return dy, dgate


def gated_add(v, gate, ve):
    """v + gate[..., None] * ve with v, ve: [B,T,H,128], gate: [B,T,H]."""
    if v.is_cuda:
        return _GatedAddFn.apply(v, gate, ve)
    return gated_add_ref(v, gate, ve)


def head_scale(y, gate):
    if y.is_cuda:
        return _HeadScaleFn.apply(y, gate)
    return head_scale_ref(y, gate)


# =============================================================================== SwiGLU (train.py:322-323)
def swiglu_ref(gf):
    h = gf.size(-1) // 2
    return F.silu(gf[..., :h]) * gf[..., h:]


class _SwiGLUFn(Function):
    @staticmethod
    def forward(ctx, gf):
        h = gf.size(-1) // 2
        gf2 = _c(gf.reshape(-1, 2 * h))
        out = torch.empty((gf2.size(0), h), dtype=torch.bfloat16, device=gf.device)
        _call("sr_swiglu_fwd", [c_void_p, c_void_p, c_long, c_int, c_void_p], gf2.data_ptr(), out.data_ptr(), gf2.size(0), h,
              _lib.stream_ptr())
        ctx.save_for_backward(gf2)
        ctx.shape = gf.shape
        return out.view(*gf.shape[:-1], h)

    @staticmethod
    def backward(ctx, d):
        (gf2,) = ctx.saved_tensors
        h = gf2.size(-1) // 2
        d2 = _c(d.reshape(-1, h))
        dgf = torch.empty_like(gf2)
        _call("sr_swiglu_bwd", [c_void_p, c_void_p, c_void_p, c_long, c_int, c_void_p], gf2.data_ptr(), d2.data_ptr(),
              dgf.data_ptr(), gf2.size(0), h, _lib.stream_ptr())
        return dgf.view(ctx.shape)


def swiglu(gf):
    """silu(gf[..., :h]) * gf[..., h:] on the output of the fused [c_gate; c_fc] projection."""
    if gf.is_cuda:
        return _SwiGLUFn.apply(gf)
    return swiglu_ref(gf)


# =============================================================================== residual + dropout (+ stochastic depth)
def dropout_add_ref(x_mid, y, p, training, x_in=None, keep=None):
    y = F.dropout(y, p, training) if p > 0 else y
    out = x_mid + y
    if x_in is not None:
        out = x_in + keep.to(out.dtype) * (out - x_in)
    return out


_dropout = {"salt": 0, "state": {}}


def next_dropout_seed() -> int:
    """Per-call-site salt: a host counter. It is baked into a captured graph; what changes between replays is the
    device-resident step counter (`dropout_state`) that every mask also hashes."""
    _dropout["salt"] += 1
    return _dropout["salt"] * 0x9E3779B1


def dropout_state(device) -> torch.Tensor:
    """int64[1] on `device`, initialised from torch's CPU generator (so torch.manual_seed governs the masks)."""
    dev = torch.device(device)
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    st = _dropout["state"].get(key)
    if st is None:
        st = torch.randint(0, 2 ** 40, (1,), dtype=torch.int64).to(dev)
        _dropout["state"][key] = st
    return st


def dropout_rng_state() -> dict:
    """Everything the dropout masks depend on besides the call arguments, for a resume file."""
    return {"salt": _dropout["salt"], "state": {k: int(v.item()) for k, v in _dropout["state"].items()}}


def set_dropout_rng_state(st: dict):
    _dropout["salt"] = int(st["salt"])
    for key, val in st["state"].items():
        dev = torch.device(key[0], key[1]) if key[0] == "cuda" else torch.device(key[0])
        if key[0] == "cuda" and not torch.cuda.is_available():
            continue
        dropout_state(dev).fill_(int(val))


def advance_dropout_state(device):
    """Call once per forward pass (inside the captured region when CUDA graphs are used)."""
    dropout_state(device).add_(1)


class _DropoutAddFn(Function):
    @staticmethod
    def forward(ctx, x_mid, y, p, seed, x_in, keep):
        x_mid, y = _c(x_mid), _c(y)
        x_in = _c(x_in) if x_in is not None else None
        out = torch.empty_like(x_mid)
        _call("sr_dropout_add_fwd", [c_void_p] * 5 + [c_long, c_float, c_ull, c_void_p, c_void_p],
              x_mid.data_ptr(), y.data_ptr(), _lib.ptr(x_in), _lib.ptr(keep), out.data_ptr(), x_mid.numel(), p, seed,
              dropout_state(x_mid.device).data_ptr(), _lib.stream_ptr())
        ctx.p, ctx.seed = p, seed
        ctx.has_in = x_in is not None
        ctx.save_for_backward(keep if keep is not None else x_mid.new_empty(0))
        return out

    @staticmethod
    def backward(ctx, g):
        (keep,) = ctx.saved_tensors
        g = _c(g)
        has_in = ctx.has_in
        dy = torch.empty_like(g)
        dmid = torch.empty_like(g) if has_in else None
        din = torch.empty_like(g) if has_in else None
        _call("sr_dropout_add_bwd", [c_void_p] * 5 + [c_long, c_float, c_ull, c_void_p, c_void_p],
              g.data_ptr(), keep.data_ptr() if has_in else 0, dy.data_ptr(), _lib.ptr(dmid), _lib.ptr(din), g.numel(),
              ctx.p, ctx.seed, dropout_state(g.device).data_ptr(), _lib.stream_ptr())
        return (dmid if has_in else g), dy, None, None, din, None


def dropout_add(x_mid, y, p, training, x_in=None, keep=None):
    """out = x_mid + dropout(y); with (x_in, keep): out = x_in + keep * (x_mid + dropout(y) - x_in)."""
    if x_mid.is_cuda:
        p_eff = float(p) if training else 0.0
        seed = next_dropout_seed() if p_eff > 0 else 0
        return _DropoutAddFn.apply(x_mid, y, p_eff, seed, x_in, keep)
    return dropout_add_ref(x_mid, y, p, training, x_in, keep)


# =============================================================================== soft-capped CE head (train.py:558-568)
def softcap_ce_ref(logits, targets, cap, vocab, weights=None, reduction="mean"):
    """logits [M, Vpad] -> per-row loss. `weights` (k,) scores row i against targets[i+k] (flattened, tiny track)."""
    z = logits[..., :vocab].float()
    if cap > 0:
        z = cap * torch.tanh(z / cap)
    M = z.size(0)
    if weights is None:
        loss = F.cross_entropy(z, targets, ignore_index=-1, reduction="none")
    else:
        lse = torch.logsumexp(z, dim=-1)
        loss = torch.zeros(M, dtype=torch.float32, device=z.device)
        for k in range(len(weights)):
            idx = torch.arange(M, device=z.device)
            valid = idx + k < M
            tk = targets[(idx + k).clamp(max=M - 1)]
            valid = valid & (tk >= 0)
            zk = z.gather(1, tk.clamp(min=0).unsqueeze(1)).squeeze(1)
            loss = loss + torch.where(valid, weights[k] * (lse - zk), torch.zeros_like(lse))
    if reduction == "none":
        return loss
    if weights is None:
        n = (targets >= 0).sum().clamp(min=1)
        return loss.sum() / n
    return loss.mean()


_CE_ARGS = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_long, c_int, c_int, c_long, c_float, c_int, c_void_p]


class _LMHeadLossFn(Function):
    """lm-head GEMM + soft-capped CE. Forward produces the logits with the tcgen05 GEMM, the CE kernel turns them into
    the (1/n scaled) logit gradient in place; backward feeds that buffer to the dX and dW GEMMs with the upstream
    scalar applied on the device. Returns the summed-and-scaled loss (mean over valid targets)."""

    @staticmethod
    def forward(ctx, x, w, grad_acc, w_t, targets, cap, vocab, weights, n_predict, mean_over_rows):
        K = x.size(-1)
        x2 = _c(x.reshape(-1, K))
        M = x2.size(0)
        logits = gemm(x2, w, b_mn=w_t)
        Vpad = logits.size(1)
        t = _c(targets.reshape(-1))
        loss_rows = torch.empty(M, dtype=torch.float32, device=x.device)
        if mean_over_rows:
            scale = torch.full((), 1.0 / M, dtype=torch.float32, device=x.device)
        else:
            scale = 1.0 / (t >= 0).sum().clamp(min=1).float()
        _call("sr_softcap_ce", _CE_ARGS, logits.data_ptr(), t.data_ptr(), loss_rows.data_ptr(), _lib.ptr(weights), n_predict,
              scale.data_ptr(), M, Vpad, vocab, logits.stride(0), cap, 1, _lib.stream_ptr())
        ctx.save_for_backward(x2, w, logits)
        ctx.grad_acc, ctx.w_t, ctx.xshape = grad_acc, w_t, x.shape
        return loss_rows.sum() * scale

    @staticmethod
    def backward(ctx, g):
        x2, w, dlogits = ctx.saved_tensors
        w_t = ctx.w_t
        g = _c(g.float())
        dx = gemm(dlogits, w, b_mn=not w_t, alpha_t=g).view(ctx.xshape) if ctx.needs_input_grad[0] else None
        acc = ctx.grad_acc
        dw = None
        if acc is not None:
            if w_t:
                gemm(x2, dlogits, out=acc, cin=acc, a_mn=True, b_mn=True, beta=1.0, alpha_t=g)
            else:
                gemm(dlogits, x2, out=acc, cin=acc, a_mn=True, b_mn=True, beta=1.0, alpha_t=g)
        elif ctx.needs_input_grad[1]:
            dw = (gemm(x2, dlogits, a_mn=True, b_mn=True, alpha_t=g) if w_t
                  else gemm(dlogits, x2, a_mn=True, b_mn=True, alpha_t=g))
        return dx, dw, None, None, None, None, None, None, None, None


# ---- fused head: the GEMM epilogue does the softcap, the row sums and the unnormalised gradient (csrc/lmhead_ce.cu)
FP8_X_SCALE = 100.0 / 448.0     # static per-tensor scales of the reference's fp8 head (tiny/train.py:187-189)
FP8_W_SCALE = 1.6 / 448.0
_head = {"fused": True}


def set_fused_head(on: bool) -> None:
    """A/B switch: True (default) = lm-head GEMM with the cross-entropy epilogue, False = GEMM -> bf16 logits ->
    separate loss kernel."""
    _head["fused"] = bool(on)


_HEAD_ARGS = [c_void_p, c_void_p, c_void_p, _lib.c_ll, c_int, c_int, c_int, _lib.c_ll, _lib.c_ll, c_int, c_int, c_float,
              c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
              c_void_p, c_void_p, _lib.c_ll, c_void_p, c_int, c_void_p, c_void_p]


def _fused_head_ok(x2, w, w_t, cap, fp8):
    K = x2.size(-1)
    N = w.size(1) if w_t else w.size(0)
    return (_head["fused"] and cap > 0 and N % 32 == 0 and K % (16 if fp8 else 8) == 0 and w.dtype == torch.bfloat16
            and w.stride(-1) == 1 and x2.dtype == torch.bfloat16)


FP8_GRAD_MULT = 256.0           # the logit gradient (in probability units, |.| <= sum of target weights) is stored as
                                # e5m2(256 * value): probabilities down to 6e-8 stay representable


def _fused_head_forward(x2, w, w_t, t, cap, vocab, weights, n_predict, mean_over_rows, fp8, want_grad):
    """Runs sr_lmhead_ce_fwd. Returns (loss scalar, loss_rows, saved) where `saved` holds what the backward needs
    (None when `want_grad` is False: evaluation allocates nothing of size [tokens, vocab] at all).
      bf16: saved = (E', rscale, Xs)                         dx = diag(rscale) E' W,  dW += E'^T Xs
      fp8 : saved = (G8, G8^T, X8^T, W8 as [d, V], scale)    both backward products on fp8 operands as well"""
    M, K = x2.shape
    N = w.size(1) if w_t else w.size(0)
    dev = x2.device
    tiles_n = (N + 255) // 256
    partials = torch.empty((tiles_n, M), dtype=torch.float32, device=dev)
    ztgt = torch.empty((M, 4), dtype=torch.float32, device=dev)
    loss_rows = torch.empty(M, dtype=torch.float32, device=dev)
    scal = torch.empty(2, dtype=torch.float32, device=dev)      # [0] = scale, [1] = loss
    E = rscale = Xs = None
    if want_grad:
        E = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        rscale = torch.empty(M, dtype=torch.float32, device=dev)
        if not fp8:
            Xs = torch.empty((M, K), dtype=torch.bfloat16, device=dev)
    if fp8:
        from .gemm import quantize_fp8
        xa = quantize_fp8(x2, FP8_X_SCALE)
        wa = quantize_fp8(w, FP8_W_SCALE, transpose=w_t)        # [N, K]
        alpha, b_mn, lda, ldb = FP8_X_SCALE * FP8_W_SCALE, 0, xa.stride(0), wa.stride(0)
    else:
        xa, wa, alpha, b_mn, lda, ldb = x2, w, 1.0, int(w_t), x2.stride(0), w.stride(0)
    _call("sr_lmhead_ce_fwd", _HEAD_ARGS, xa.data_ptr(), wa.data_ptr(), _lib.ptr(E), N, M, N, K, lda, ldb, b_mn, int(fp8),
          alpha, t.data_ptr(), _lib.ptr(weights), n_predict, vocab, cap, int(mean_over_rows), scal.data_ptr(),
          partials.data_ptr(), ztgt.data_ptr(), loss_rows.data_ptr(), scal.data_ptr() + 4, _lib.ptr(rscale),
          x2.data_ptr(), x2.stride(0), _lib.ptr(Xs), 0, _lib.status_buffer(dev).data_ptr(), _lib.stream_ptr())
    if not want_grad:
        return scal[1], loss_rows, None
    if not fp8:
        return scal[1], loss_rows, (E, rscale, Xs)
    # fp8 backward operands, every one K-major: the gradient in both layouts (one pass over E'), x^T, and W as [d, V]
    from .gemm import fp8_empty
    G8 = fp8_empty((M, N), torch.float8_e5m2, dev)
    G8T = fp8_empty((N, M), torch.float8_e5m2, dev)
    _call("sr_quant_fp8_dual", [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_long, c_int, c_long, c_long, c_long,
                                c_int, c_void_p],
          E.data_ptr(), rscale.data_ptr(), scal.data_ptr(), FP8_GRAD_MULT, G8.data_ptr(), G8T.data_ptr(), M, N, E.stride(0),
          G8.stride(0), G8T.stride(0), 1, _lib.stream_ptr())
    del E
    X8T = quantize_fp8(x2, FP8_X_SCALE, transpose=True)         # [K, M]
    Wd = quantize_fp8(w, FP8_W_SCALE, transpose=not w_t)        # [K, N]: the B operand of dx = G W
    return scal[1], loss_rows, (G8, G8T, X8T, Wd, scal[0:1])


class _FusedLMHeadLossFn(Function):
    """lm-head + soft-capped CE on the fused kernel: forward leaves E' (bf16, the logit gradient up to the per-row
    factor `rscale`) and the pre-scaled activations; backward is dx = diag(rscale) E' W (row factor in the GEMM
    epilogue) and dW += E'^T (rscale * x), both scaled by the upstream scalar on the device. With `fp8` the forward
    product runs on e4m3 operands and the two backward products on the e5m2 gradient and e4m3 x / W (the precision
    recipe of the reference's tiny track, tiny/cuda_kernels.py:338-414), each with fp32 accumulation."""

    @staticmethod
    def forward(ctx, x, w, grad_acc, w_t, targets, cap, vocab, weights, n_predict, mean_over_rows, fp8):
        K = x.size(-1)
        x2 = _c(x.reshape(-1, K))
        t = _c(targets.reshape(-1))
        loss, _, saved = _fused_head_forward(x2, w, w_t, t, cap, vocab, weights, n_predict, mean_over_rows, fp8, True)
        ctx.save_for_backward(*saved)
        ctx.grad_acc, ctx.w_t, ctx.xshape, ctx.fp8, ctx.w = grad_acc, w_t, x.shape, fp8, (None if fp8 else w)
        return loss

    @staticmethod
    def backward(ctx, g):
        w_t, acc = ctx.w_t, ctx.grad_acc
        g = _c(g.float())
        dx = dw = None
        if ctx.fp8:
            from .gemm import gemm_fp8
            G8, G8T, X8T, Wd, scale = ctx.saved_tensors
            gs = (g * scale).reshape(())                        # upstream scalar times 1 / #tokens, on the device
            if ctx.needs_input_grad[0]:
                dx = gemm_fp8(G8, Wd, alpha=FP8_W_SCALE / FP8_GRAD_MULT, alpha_t=gs).view(ctx.xshape)
            a = FP8_X_SCALE / FP8_GRAD_MULT
            if acc is not None:
                if w_t:
                    gemm_fp8(X8T, G8T, out=acc, cin=acc, alpha=a, beta=1.0, alpha_t=gs)
                else:
                    gemm_fp8(G8T, X8T, out=acc, cin=acc, alpha=a, beta=1.0, alpha_t=gs)
            elif ctx.needs_input_grad[1]:
                dw = gemm_fp8(X8T, G8T, alpha=a, alpha_t=gs) if w_t else gemm_fp8(G8T, X8T, alpha=a, alpha_t=gs)
            return (dx, dw) + (None,) * 9
        E, rscale, Xs = ctx.saved_tensors
        w = ctx.w
        if ctx.needs_input_grad[0]:
            dx = gemm(E, w, b_mn=not w_t, alpha_t=g, row_scale=rscale).view(ctx.xshape)
        if acc is not None:
            if w_t:
                gemm(Xs, E, out=acc, cin=acc, a_mn=True, b_mn=True, beta=1.0, alpha_t=g)
            else:
                gemm(E, Xs, out=acc, cin=acc, a_mn=True, b_mn=True, beta=1.0, alpha_t=g)
        elif ctx.needs_input_grad[1]:
            dw = (gemm(Xs, E, a_mn=True, b_mn=True, alpha_t=g) if w_t else gemm(E, Xs, a_mn=True, b_mn=True, alpha_t=g))
        return (dx, dw) + (None,) * 9


def lm_head_loss(x, w, targets, cap, vocab, grad_acc=None, w_t=False, weights=None, fp8=False):
    """Mean soft-capped CE of (x @ W^T)[..., :vocab] against targets (ignore_index -1).
    With `weights` (fp32 tensor of k entries) row i is scored against targets[i..i+k-1] of the flattened batch and the
    mean runs over all rows (the tiny track's shared-head multi-token loss, tiny/train.py:682-696).
    `fp8`: all three products on fp8 operands (e4m3 x and W with the reference's static per-tensor scales, e5m2 logit
    gradient; tiny/cuda_kernels.py:340-412), fp32 accumulation."""
    if x.is_cuda:
        npred = 1 if weights is None else int(weights.numel())
        wts = None if weights is None else _c(weights.float())
        x2 = x.reshape(-1, x.size(-1))
        if _fused_head_ok(x2, w, w_t, float(cap), fp8):
            return _FusedLMHeadLossFn.apply(x, w, grad_acc, w_t, targets, float(cap), int(vocab), wts, npred,
                                            weights is not None, bool(fp8))
        return _LMHeadLossFn.apply(x, w, grad_acc, w_t, targets, float(cap), int(vocab), wts, npred, weights is not None)
    logits = (x @ w.to(x.dtype)) if w_t else F.linear(x, w.to(x.dtype))
    return softcap_ce_ref(logits.reshape(-1, logits.size(-1)), targets.reshape(-1), cap, vocab, weights)


def lm_head_rows(x, w, targets, cap, vocab, w_t=False):
    """Per-token soft-capped CE (no gradient): the eval path (train.py:856)."""
    if x.is_cuda:
        K = x.size(-1)
        x2 = _c(x.reshape(-1, K))
        t = _c(targets.reshape(-1))
        if _fused_head_ok(x2, w, w_t, float(cap), False):
            return _fused_head_forward(x2, w, w_t, t, float(cap), int(vocab), None, 1, False, False, False)[1]
        logits = gemm(x2, w, b_mn=w_t)
        loss_rows = torch.empty(x2.size(0), dtype=torch.float32, device=x.device)
        _call("sr_softcap_ce", _CE_ARGS, logits.data_ptr(), t.data_ptr(), loss_rows.data_ptr(), 0, 1, 0, x2.size(0),
              logits.size(1), vocab, logits.stride(0), float(cap), 0, _lib.stream_ptr())
        return loss_rows
    logits = (x @ w.to(x.dtype)) if w_t else F.linear(x, w.to(x.dtype))
    return softcap_ce_ref(logits.reshape(-1, logits.size(-1)), targets.reshape(-1), cap, vocab, None, "none")


def lm_head_logits_grad(x, w, cap, vocab, grad_acc=None, w_t=False):
    """Differentiable soft-capped fp32 logits (distillation / label-smoothing paths, unlimited/train.py:603-634)."""
    logits = linear(x, w, grad_acc, w_t)[..., :vocab].float()
    return cap * torch.tanh(logits / cap) if cap > 0 else logits


def lm_head_logits(x, w, cap, vocab, w_t=False):
    """Soft-capped fp32 logits [..., vocab] (train.py:559-562)."""
    if x.is_cuda:
        x2 = _c(x.reshape(-1, x.size(-1)))
        logits = gemm(x2, w, b_mn=w_t).view(*x.shape[:-1], -1)
    else:
        logits = (x @ w.to(x.dtype)) if w_t else F.linear(x, w.to(x.dtype))
    logits = logits[..., :vocab].float()
    return cap * torch.tanh(logits / cap) if cap > 0 else logits


# =============================================================================== attention (train.py:211-213, 307)
def attention_ref(q, k, v, window, scale=None):
    """Causal sliding-window attention, (B,T,H,D) layout; key j visible to query i iff i-window <= j <= i."""
    B, T, H, D = q.shape
    q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if window is None or window < 0 or window >= T:
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale)
    else:
        i = torch.arange(T, device=q.device).unsqueeze(1)
        j = torch.arange(T, device=q.device).unsqueeze(0)
        mask = (j <= i) & ((i - j) <= window)
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, scale=scale)
    return y.transpose(1, 2)


_attn_impl = {"fn": None}


def set_attention_impl(fn):
    """Install the CUDA attention implementation: fn(q, k, v, window, scale) -> y, all (B,T,H,D) bf16."""
    _attn_impl["fn"] = fn


def attention(q, k, v, window, scale=None):
    if q.is_cuda and _attn_impl["fn"] is not None:
        return _attn_impl["fn"](q, k, v, window, scale)
    return attention_ref(q, k, v, window, scale)
