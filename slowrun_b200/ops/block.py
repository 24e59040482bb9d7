"""The transformer block (with its lambda-mix prologue) as ONE autograd node with a hand-written backward.

Forward and backward are straight-line sequences of the sm_100a kernels: tcgen05 GEMMs for the five projections
(weight gradients accumulate into the fp32 arenas inside the GEMM epilogue), fused row-wise kernels in between, the
attention implementation through its explicit fwd/bwd interface. Every gradient tensor is written once, by the
kernel that produces it; autograd only sees the three activations entering the block (previous residual stream, x0,
U-Net skip). Semantics are those of the reference block (train.py:282-344, 514-525): value residual gated per head,
RoPE then QK-norm, per-head sigmoid attention gate, IHA weight mixing, SwiGLU, dropout on both residual branches,
stochastic depth as a blend with the block input.
"""
from __future__ import annotations

import torch
from torch.autograd import Function

from . import _lib
from . import functional as ops
from .attention import current_impl
from .gemm import gemm

P, I, L, F32, ULL = _lib.c_void_p, _lib.c_int, _lib.ctypes.c_long, _lib.c_float, _lib.ctypes.c_ulonglong


def _call(name, argtypes, *args):
    rc = _lib.fn(name, argtypes)(*args)
    if rc != 0:
        raise RuntimeError(f"{name}: launcher returned {rc}")


def _sp():
    return torch.cuda.current_stream().cuda_stream


def _rmsnorm_fwd(x, eps):
    y = torch.empty_like(x)
    _call("sr_rmsnorm_fwd", [P, P, L, I, L, F32, P], x.data_ptr(), y.data_ptr(), x.size(0), x.size(1), x.stride(0), eps, _sp())
    return y


def _rmsnorm_bwd(x, dy, dres, eps):
    dx = torch.empty_like(x)
    _call("sr_rmsnorm_bwd", [P, P, P, P, L, I, L, F32, P], x.data_ptr(), dy.data_ptr(), _lib.ptr(dres), dx.data_ptr(),
          x.size(0), x.size(1), x.stride(0), eps, _sp())
    return dx


def _dropout_add_fwd(x_mid, y, p, seed, x_in=None, keep=None):
    out = torch.empty_like(x_mid)
    _call("sr_dropout_add_fwd", [P] * 5 + [L, F32, ULL, P, P], x_mid.data_ptr(), y.data_ptr(), _lib.ptr(x_in), _lib.ptr(keep),
          out.data_ptr(), x_mid.numel(), p, seed, ops.dropout_state(x_mid.device).data_ptr(), _sp())
    return out


def _dropout_add_bwd(g, p, seed, keep=None):
    dy = torch.empty_like(g)
    dmid = torch.empty_like(g) if keep is not None else None
    din = torch.empty_like(g) if keep is not None else None
    _call("sr_dropout_add_bwd", [P] * 5 + [L, F32, ULL, P, P], g.data_ptr(), _lib.ptr(keep), dy.data_ptr(), _lib.ptr(dmid),
          _lib.ptr(din), g.numel(), p, seed, ops.dropout_state(g.device).data_ptr(), _sp())
    return dy, dmid, din


def iha_mix_weights(mixes, w16, H):
    """W'[p] = bf16(mix[p]) @ W[p].view(H, -1); falls back to a library bmm for head counts without a kernel."""
    Pn = mixes.size(0)
    J = w16.numel() // (Pn * H)
    out = torch.empty_like(w16)
    rc = _lib.fn("sr_iha_mix_fwd", [P, P, P, I, I, L, P])(mixes.data_ptr(), w16.data_ptr(), out.data_ptr(), Pn, H, J, _sp())
    if rc == -7:
        return torch.bmm(mixes.to(torch.bfloat16), w16.view(Pn, H, J)).view(w16.shape)
    if rc != 0:
        raise RuntimeError(f"sr_iha_mix_fwd: launcher returned {rc}")
    return out


def _stacked_mixes(model, attn, H, device):
    """([3, H, H] fp32 mixing matrices, [3, H, H] view of their gradient accumulators or None). The three matrices of a
    layer sit next to each other in the flat small-parameter arena, so both are views and nothing is launched; a model
    without that layout (no v mix, unequal head counts) gets a stacked copy."""
    arena = getattr(model, "arena", None)
    if arena is not None and attn.iha_mix_v:
        offs = [arena.small_offsets.get(id(p)) for p in (attn.q_mix, attn.k_mix, attn.v_mix)]
        n = H * H
        if all(o is not None and o[1] == n for o in offs) and offs[1][0] == offs[0][0] + n and offs[2][0] == offs[1][0] + n:
            a0 = offs[0][0]
            gacc = arena.small_grads[a0:a0 + 3 * n].view(3, H, H)
            if attn.q_mix.grad is None or attn.q_mix.grad.data_ptr() != gacc.data_ptr():
                gacc = None                     # the parameter's .grad no longer aliases the arena
            return arena.small_P[a0:a0 + 3 * n].view(3, H, H), gacc
    third = attn.v_mix.data if attn.iha_mix_v else torch.eye(H, device=device, dtype=torch.float32)
    return torch.stack([attn.q_mix.data, attn.k_mix.data, third]), None


def iha_mix_backward(mixes, w16, dwp, grad_w, H, dmix_acc=None):
    """grad_w (fp32) += bf16(mix)^T @ dW'; returns dmix [P, H, H] fp32, or adds it into `dmix_acc` and returns None."""
    Pn = mixes.size(0)
    J = w16.numel() // (Pn * H)
    if dmix_acc is not None and J % 8 == 0:
        rc = _lib.fn("sr_iha_mix_bwd", [P, P, P, P, P, I, I, L, P])(mixes.data_ptr(), w16.data_ptr(), dwp.data_ptr(),
                                                                   grad_w.data_ptr(), 0, Pn, H, J, _sp())
        if rc == 0:
            gemm(dwp.view(Pn, H, J), w16.view(Pn, H, J), out=dmix_acc, cin=dmix_acc, beta=1.0, bn=128)
            return None
        if rc != -7:
            raise RuntimeError(f"sr_iha_mix_bwd: launcher returned {rc}")
    dmix = torch.zeros_like(mixes)
    # dmix[p] = dW'[p] W[p]^T: a [H x J] x [J x H] product with a very long K, done by the split-K tcgen05 GEMM
    # (every CTA takes a share of K and adds its partial H x H tile)
    use_gemm = J % 8 == 0
    rc = _lib.fn("sr_iha_mix_bwd", [P, P, P, P, P, I, I, L, P])(mixes.data_ptr(), w16.data_ptr(), dwp.data_ptr(),
                                                               grad_w.data_ptr(), 0 if use_gemm else dmix.data_ptr(),
                                                               Pn, H, J, _sp())
    if rc == 0 and use_gemm:
        gemm(dwp.view(Pn, H, J), w16.view(Pn, H, J), out=dmix, cin=dmix, beta=1.0, bn=128)
    if rc == -7:
        d3 = dwp.view(Pn, H, J)
        m16 = mixes.to(torch.bfloat16)
        dmix = torch.bmm(d3, w16.view(Pn, H, J).transpose(1, 2)).float()
        grad_w.view(Pn, H, J).add_(torch.bmm(m16.transpose(1, 2), d3))
        return dmix
    if rc != 0:
        raise RuntimeError(f"sr_iha_mix_bwd: launcher returned {rc}")
    return dmix


def _gate_fwd(a, w, H, nc, scale):
    """[M, H] fp32 gate = scale * sigmoid(a[:, :nc] @ bf16(w)^T), the bf16-autocast linear + sigmoid of the reference."""
    M = a.size(0)
    gate = torch.empty((M, H), dtype=torch.float32, device=a.device)
    _call("sr_gate_fwd", [P, L, P, P, L, I, I, F32, P], a.data_ptr(), a.stride(0), w.data_ptr(), gate.data_ptr(), M, H, nc,
          scale, _sp())
    return gate


def _gate_bwd(dgate, gate, a, w_param, da, H, nc, scale):
    """Adds the gate linear's weight gradient into w_param.grad (fp32) and its input gradient into da[:, :nc]."""
    _call("sr_gate_bwd", [P, P, P, L, P, P, P, L, L, I, I, F32, P], dgate.data_ptr(), gate.data_ptr(), a.data_ptr(),
          a.stride(0), w_param.data.data_ptr(), w_param.grad.data_ptr(), da.data_ptr(), da.stride(0), a.size(0), H, nc,
          scale, _sp())


class _BlockFn(Function):
    @staticmethod
    def forward(ctx, x_prev, x0, skip, model, block, i, j, do_mix, ve_lin, window, scale, training):
        B, T, C = x_prev.shape
        M = B * T
        attn, mlp = block.attn, block.mlp
        H, D = attn.n_head, attn.head_dim
        eps = float(model.norm_eps)
        impl = current_impl()
        xp = x_prev.reshape(M, C)
        xp = xp if xp.is_contiguous() else xp.contiguous()
        x0_2 = None
        if x0 is not None:
            x0_2 = x0.reshape(M, C)
            x0_2 = x0_2 if x0_2.is_contiguous() else x0_2.contiguous()
        sk = None
        if skip is not None:
            sk = skip.reshape(M, C)
            sk = sk if sk.is_contiguous() else sk.contiguous()
        # ---- lambda mix
        if do_mix:
            x, a = torch.empty_like(xp), torch.empty_like(xp)
            rl, xl, sw = model.resid_lambdas, model.x0_lambdas, model.skip_weights
            _call("sr_mix_norm_fwd", [P] * 8 + [L, I, F32, P], xp.data_ptr(), x0_2.data_ptr(), _lib.ptr(sk), x.data_ptr(),
                  a.data_ptr(), rl.data_ptr() + 4 * i, xl.data_ptr() + 4 * i, sw.data_ptr() + 4 * j if sk is not None else 0,
                  M, C, eps, _sp())
        else:
            x = xp
            a = _rmsnorm_fwd(x, eps)
        # ---- projections
        ve = gemm(x0_2, ve_lin.fused["w16"]) if ve_lin is not None else None
        fz = attn.fused
        mixes = None
        if attn.use_iha:
            mixes, _ = _stacked_mixes(model, attn, H, x.device)
            w_qkv = iha_mix_weights(mixes, fz["qkv_w16"], H)
        else:
            w_qkv = fz["qkv_w16"]
        qkv = gemm(a, w_qkv)
        # ---- gates (tiny [M, H] tensors: library ops)
        agate = _gate_fwd(a, attn.attn_gate.weight.data, H, attn.attn_gate_channels, 1.0)
        ve_gate = _gate_fwd(a, attn.ve_gate.weight.data, H, attn.ve_gate_channels, 2.0) if ve is not None else None
        # ---- split + value residual + RoPE + QK norm
        cos, sin = model.rotary.cos, model.rotary.sin
        cos2, sin2 = cos.view(-1, cos.size(-1)), sin.view(-1, sin.size(-1))
        q = torch.empty((B, T, H, D), dtype=torch.bfloat16, device=x.device)
        k, v = torch.empty_like(q), torch.empty_like(q)
        koff = int(bool(attn.use_key_offset) and T > 1)
        _call("sr_qkv_prep_fwd", [P] * 8 + [L, I, I, F32, I, P], qkv.data_ptr(), _lib.ptr(ve), _lib.ptr(ve_gate), cos2.data_ptr(),
              sin2.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), M, H, T, eps, koff, _sp())
        y, attn_saved = impl.fwd(q, k, v, window, scale)
        y2 = torch.empty_like(y)
        xsa = model.xsa_alphas if (do_mix and model._xsa_enabled(i)) else None     # [n_layer, H] fp32, row i
        _call("sr_attn_post_fwd", [P] * 5 + [L, I, F32, P], y.data_ptr(), v.data_ptr(), agate.data_ptr(),
              xsa.data_ptr() + 4 * i * H if xsa is not None else 0, y2.data_ptr(), M, H, float(attn.xsa_eps), _sp())
        o = gemm(y2.view(M, C), fz["proj_w16"])
        # ---- residual, MLP
        p_attn = float(attn.dropout) if training else 0.0
        p_mlp = float(mlp.dropout) if training else 0.0
        seed1 = ops.next_dropout_seed() if p_attn > 0 else 0
        seed2 = ops.next_dropout_seed() if p_mlp > 0 else 0
        x_mid, n = torch.empty_like(x), torch.empty_like(x)
        _call("sr_add_norm_fwd", [P] * 4 + [L, I, F32, F32, ULL, P, P], x.data_ptr(), o.data_ptr(), x_mid.data_ptr(), n.data_ptr(),
              M, C, eps, p_attn, seed1, ops.dropout_state(x.device).data_ptr(), _sp())
        mz = mlp.fused
        gf = gemm(n, mz["gf_w16"])
        hdim = gf.size(1) // 2
        hdn = torch.empty((M, hdim), dtype=torch.bfloat16, device=x.device)
        _call("sr_swiglu_fwd", [P, P, L, I, P], gf.data_ptr(), hdn.data_ptr(), M, hdim, _sp())
        mo = gemm(hdn, mz["proj_w16"])
        keep = None
        if training and block.drop_prob > 0:
            keep = (torch.rand((), device=x.device) >= block.drop_prob).float()
            out = _dropout_add_fwd(x_mid, mo, p_mlp, seed2, x_in=x, keep=keep)
        else:
            out = _dropout_add_fwd(x_mid, mo, p_mlp, seed2)
        ctx.save_for_backward(xp, x0_2 if x0_2 is not None else xp.new_empty(0), sk if sk is not None else xp.new_empty(0))
        ctx.t = (x, a, ve, mixes, w_qkv, qkv, agate, ve_gate, attn_saved, y, y2, x_mid, n, gf, hdn, keep, v, xsa, koff)
        ctx.meta = (model, block, i, j, do_mix, ve_lin, p_attn, p_mlp, seed1, seed2, eps, impl, (B, T, C, H, D),
                    x0 is not None, skip is not None)
        return out.view(B, T, C)

    @staticmethod
    def backward(ctx, g_out):
        xp, x0_2, sk = ctx.saved_tensors
        x, a, ve, mixes, w_qkv, qkv, agate, ve_gate, attn_saved, y, y2, x_mid, n, gf, hdn, keep, v, xsa, koff = ctx.t
        model, block, i, j, do_mix, ve_lin, p_attn, p_mlp, seed1, seed2, eps, impl, dims, has_x0, has_skip = ctx.meta
        ctx.t = None
        B, T, C, H, D = dims
        M = B * T
        attn, mlp = block.attn, block.mlp
        fz, mz = attn.fused, mlp.fused
        g = g_out.reshape(M, C)
        g = g if g.is_contiguous() else g.contiguous()
        # ---- MLP branch
        dmo, g_mid, g_in = _dropout_add_bwd(g, p_mlp, seed2, keep)
        if keep is None:
            g_mid = g
        dhdn = gemm(dmo, mz["proj_w16"], b_mn=True)
        gemm(dmo, hdn, out=mz["proj_grad"], cin=mz["proj_grad"], a_mn=True, b_mn=True, beta=1.0)
        dgf = torch.empty_like(gf)
        _call("sr_swiglu_bwd", [P, P, P, L, I, P], gf.data_ptr(), dhdn.data_ptr(), dgf.data_ptr(), M, gf.size(1) // 2, _sp())
        dn = gemm(dgf, mz["gf_w16"], b_mn=True)
        gemm(dgf, n, out=mz["gf_grad"], cin=mz["gf_grad"], a_mn=True, b_mn=True, beta=1.0)
        # ---- attention branch: norm backward + residual gradient + gradient of the dropped branch in one pass
        g_mid_tot, do = torch.empty_like(x_mid), torch.empty_like(x_mid)
        _call("sr_norm_bwd_drop", [P] * 5 + [L, I, F32, F32, ULL, P, P], x_mid.data_ptr(), dn.data_ptr(), g_mid.data_ptr(),
              g_mid_tot.data_ptr(), do.data_ptr(), M, C, eps, p_attn, seed1, ops.dropout_state(g.device).data_ptr(), _sp())
        dy2 = gemm(do, fz["proj_w16"], b_mn=True)
        gemm(do, y2.view(M, C), out=fz["proj_grad"], cin=fz["proj_grad"], a_mn=True, b_mn=True, beta=1.0)
        dy = torch.empty_like(y)
        dagate = torch.empty((M, H), dtype=torch.float32, device=g.device)
        fused_attn_bwd = getattr(impl, "has_bwd", False) and hasattr(impl, "bwd_fused")
        # gate (and exclusive self-attention) backward; it already forms delta = rowsum(dy * y) for the attention
        # backward, which in turn leaves dQ in fp32 for qkv_prep_bwd
        delta = torch.empty((B, H, T), dtype=torch.float32, device=g.device)
        dv_x = torch.empty_like(y) if xsa is not None else None
        _call("sr_attn_post_bwd", [P] * 10 + [L, I, I, F32, P], dy2.data_ptr(), y.data_ptr(), v.data_ptr(), agate.data_ptr(),
              xsa.data_ptr() + 4 * i * H if xsa is not None else 0, dy.data_ptr(), dagate.data_ptr(), delta.data_ptr(),
              _lib.ptr(dv_x), xsa.grad.data_ptr() + 4 * i * H if xsa is not None else 0, M, H, T, float(attn.xsa_eps), _sp())
        if fused_attn_bwd:
            dq, dk, dv = impl.bwd_fused(attn_saved, dy, delta)
        else:
            dq, dk, dv = impl.bwd(attn_saved, dy)
        dqkv = torch.empty_like(qkv)
        dve = torch.empty((M, C), dtype=torch.bfloat16, device=g.device) if ve is not None else None
        dvegate = torch.empty((M, H), dtype=torch.float32, device=g.device) if ve is not None else None
        cos, sin = model.rotary.cos, model.rotary.sin
        cos2, sin2 = cos.view(-1, cos.size(-1)), sin.view(-1, sin.size(-1))
        _call("sr_qkv_prep_bwd_f32dq" if fused_attn_bwd else "sr_qkv_prep_bwd", [P] * 11 + [L, I, I, F32, I, P, P], qkv.data_ptr(),
              _lib.ptr(ve), _lib.ptr(ve_gate), cos2.data_ptr(), sin2.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
              dqkv.data_ptr(), _lib.ptr(dve), _lib.ptr(dvegate), M, H, T, eps, koff, _lib.ptr(dv_x), _sp())
        da = gemm(dqkv, w_qkv, b_mn=True)
        if mixes is not None:
            dwp = gemm(dqkv, a, a_mn=True, b_mn=True)
            _, dmix_acc = _stacked_mixes(model, attn, H, x.device)
            dmix = iha_mix_backward(mixes, fz["qkv_w16"], dwp, fz["qkv_grad"], H, dmix_acc)
            if dmix is not None:
                attn.q_mix.grad.add_(dmix[0])
                attn.k_mix.grad.add_(dmix[1])
                if attn.iha_mix_v:
                    attn.v_mix.grad.add_(dmix[2])
        else:
            gemm(dqkv, a, out=fz["qkv_grad"], cin=fz["qkv_grad"], a_mn=True, b_mn=True, beta=1.0)
        # ---- gates (tiny)
        _gate_bwd(dagate, agate, a, attn.attn_gate.weight, da, H, attn.attn_gate_channels, 1.0)
        dx0 = None
        if ve is not None:
            _gate_bwd(dvegate, ve_gate, a, attn.ve_gate.weight, da, H, attn.ve_gate_channels, 2.0)
            gemm(dve, x0_2, out=ve_lin.fused["grad"], cin=ve_lin.fused["grad"], a_mn=True, b_mn=True, beta=1.0)
        # ---- back through the first norm and the lambda mix
        if not do_mix:
            if g_in is not None:
                g_mid_tot.add_(g_in)
            g_x = _rmsnorm_bwd(x, da, g_mid_tot, eps)
            if ve is not None:
                dx0 = gemm(dve, ve_lin.fused["w16"], b_mn=True)
            return (g_x.view(B, T, C), dx0.view(B, T, C) if dx0 is not None else None, None) + (None,) * 9
        dxp = torch.empty_like(x)
        dx0 = torch.empty_like(x)
        dsk = torch.empty_like(x) if has_skip else None
        rl, xl, sw = model.resid_lambdas, model.x0_lambdas, model.skip_weights
        # the three scalar gradients are accumulated straight into the (fp32, arena-backed) .grad entries
        _call("sr_norm_bwd_mix", [P] * 16 + [L, I, F32, P], x.data_ptr(), da.data_ptr(), g_mid_tot.data_ptr(), _lib.ptr(g_in),
              xp.data_ptr(), x0_2.data_ptr(), sk.data_ptr() if has_skip else 0, dxp.data_ptr(), dx0.data_ptr(), _lib.ptr(dsk),
              rl.data_ptr() + 4 * i, xl.data_ptr() + 4 * i, sw.data_ptr() + 4 * j if has_skip else 0,
              rl.grad.data_ptr() + 4 * i, xl.grad.data_ptr() + 4 * i, sw.grad.data_ptr() + 4 * j if has_skip else 0,
              M, C, eps, _sp())
        if ve is not None:
            gemm(dve, ve_lin.fused["w16"], out=dx0, cin=dx0, b_mn=True, beta=1.0)
        return (dxp.view(B, T, C), dx0.view(B, T, C), dsk.view(B, T, C) if dsk is not None else None) + (None,) * 9


def block_forward(model, block, x_prev, x0, skip, i, j, do_mix, ve_lin, window, scale):
    """x_out of layer `i` (lambda mix with skip j when do_mix, then the block) through the fused autograd node."""
    return _BlockFn.apply(x_prev, x0, skip, model, block, i, j, do_mix, ve_lin, window[0], scale, model.training)


def block_supported(model, block) -> bool:
    """The fused node covers every block of the four tracks (head_dim 128, weights large enough to have bf16 shadows);
    anything else goes through the op-by-op path of `GPT._block_forward`."""
    a = block.attn
    if getattr(a, "is_linear_attention", False):
        return False
    return a.head_dim == 128 and a.n_head <= 64 and a.fused is not None and a.fused["qkv_w16"] is not None
