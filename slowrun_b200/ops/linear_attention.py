"""Gated delta rule: the token mixer of the hybrid research fork (Gated DeltaNet and Kimi Delta Attention layers).

Per head, with a fast-weight state S of shape [Dk, Dv]:
    S <- diag(exp(g_t)) S ;   r = v_t - S^T k_t ;   S <- S + beta_t k_t r^T ;   o_t = S^T q_t
`g` is a log-decay <= 0, one per head ([B, T, H], Gated DeltaNet) or one per key channel ([B, T, H, Dk], Kimi Delta
Attention). The reference fork delegates this to flash-linear-attention's Triton kernels
(research/hybrid_attn/train.py:36-38, 459-468, 612-628). Three statements of the same function live here:

* `gated_delta_rule_recurrent`  the definition, token by token in fp32: the numerics oracle;
* `gated_delta_rule_chunked`    chunk-parallel form in plain PyTorch (differentiable, any device): inside a chunk the
                                writes are obtained from one unit-lower-triangular solve, chunks are chained through
                                the state. Every exponential is of a non-positive number, so it is safe for any decay;
* `gated_delta_rule`            the op the model calls: on a GPU the forward runs the CUDA recurrence kernel
                                (csrc/gated_delta.cu, state in registers) and the backward re-derives the gradients from
                                the chunked form; elsewhere it is the chunked form throughout.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch.autograd import Function


def _expand_decay(g, Dk):
    """[B, T, H] or [B, T, H, Dk] -> [B, T, H, Dk] fp32"""
    g = g.float()
    return g.unsqueeze(-1).expand(*g.shape, Dk) if g.dim() == 3 else g


def gated_delta_rule_recurrent(q, k, v, g, beta, initial_state=None, return_state=False):
    """q, k: [B, T, H, Dk]; v: [B, T, H, Dv]; g: log-decay [B, T, H] or [B, T, H, Dk]; beta: [B, T, H].
    Returns o [B, T, H, Dv] in v's dtype (and the final state [B, H, Dk, Dv] when asked)."""
    B, T, H, Dk = q.shape
    Dv = v.size(-1)
    S = torch.zeros(B, H, Dk, Dv, dtype=torch.float32, device=q.device) if initial_state is None else initial_state.float()
    qf, kf, vf, bf = q.float(), k.float(), v.float(), beta.float()
    d = torch.exp(_expand_decay(g, Dk))
    out = []
    for t in range(T):
        S = S * d[:, t].unsqueeze(-1)
        r = vf[:, t] - torch.einsum("bhkv,bhk->bhv", S, kf[:, t])
        S = S + bf[:, t][..., None, None] * kf[:, t].unsqueeze(-1) * r.unsqueeze(-2)
        out.append(torch.einsum("bhkv,bhk->bhv", S, qf[:, t]))
    o = torch.stack(out, dim=1).to(v.dtype)
    return (o, S) if return_state else o


def gated_delta_rule_chunked(q, k, v, g, beta, chunk_size=None, initial_state=None, return_state=False):
    """Same function, chunk by chunk. With G_t the running sum of g inside the chunk, S0 the state entering it:
        A[t, j] = beta_j sum_c k_t[c] k_j[c] exp(G_t[c] - G_j[c])          j <  t   (strictly lower triangular)
        P[t, j] = beta_j sum_c q_t[c] k_j[c] exp(G_t[c] - G_j[c])          j <= t
        R = (I + A)^-1 (V - (exp(G) * K) S0)                               the writes r_t of the whole chunk
        O = (exp(G) * Q) S0 + P R
        S_end = exp(G_C) * S0 + sum_j exp(G_C - G_j) * beta_j k_j r_j^T
    A per-head decay makes exp(G_t - G_j) a [C, C] matrix; a per-channel decay needs the [C, C, Dk] tensor, for which
    the chunk is kept short."""
    B, T, H, Dk = q.shape
    Dv = v.size(-1)
    per_channel = g.dim() == 4
    C = chunk_size or (16 if per_channel else 64)
    pad = (-T) % C
    qf, kf, vf, bf, gf = q.float(), k.float(), v.float(), beta.float(), g.float()
    if pad:
        qf, kf, vf = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (qf, kf, vf))
        bf = F.pad(bf, (0, 0, 0, pad))                       # beta = 0: padded tokens write nothing
        gf = F.pad(gf, (0, 0, 0, 0, 0, pad)) if per_channel else F.pad(gf, (0, 0, 0, pad))
    n = (T + pad) // C
    # [B, H, n, C, D] layout
    def heads(t):
        return t.view(B, n, C, H, -1).permute(0, 3, 1, 2, 4)
    Q, K, V = heads(qf), heads(kf), heads(vf)
    Bt = bf.view(B, n, C, H).permute(0, 3, 1, 2)                               # [B, H, n, C]
    Gc = torch.cumsum(heads(gf) if per_channel else gf.view(B, n, C, H).permute(0, 3, 1, 2), dim=3)
    lower = torch.tril(torch.ones(C, C, dtype=torch.bool, device=q.device))
    strict = torch.tril(torch.ones(C, C, dtype=torch.bool, device=q.device), -1)
    if per_channel:
        # E[t, j, c] = exp(G_t[c] - G_j[c]) on and below the diagonal, 0 above (the difference is <= 0 there)
        diff = (Gc.unsqueeze(4) - Gc.unsqueeze(3)).masked_fill(~lower[..., None], float("-inf"))
        E = torch.exp(diff)                                                     # [B, H, n, C, C, Dk]
        KK = torch.einsum("bhntc,bhnjc,bhntjc->bhntj", K, K, E)
        QK = torch.einsum("bhntc,bhnjc,bhntjc->bhntj", Q, K, E)
        Dt = torch.exp(Gc)                                                      # [B, H, n, C, Dk]
        Dend = torch.exp(Gc[:, :, :, -1:, :] - Gc)                              # exp(G_C - G_j) per channel
    else:
        diff = (Gc.unsqueeze(4) - Gc.unsqueeze(3)).masked_fill(~lower, float("-inf"))
        E = torch.exp(diff)                                                     # [B, H, n, C, C]
        KK = torch.einsum("bhntc,bhnjc->bhntj", K, K) * E
        QK = torch.einsum("bhntc,bhnjc->bhntj", Q, K) * E
        Dt = torch.exp(Gc).unsqueeze(-1)                                        # [B, H, n, C, 1]
        Dend = torch.exp(Gc[:, :, :, -1:] - Gc).unsqueeze(-1)
    A = (KK * Bt.unsqueeze(3)).masked_fill(~strict, 0.0)
    P = (QK * Bt.unsqueeze(3)).masked_fill(~lower, 0.0)
    eye = torch.eye(C, dtype=torch.float32, device=q.device)
    S = torch.zeros(B, H, Dk, Dv, dtype=torch.float32, device=q.device) if initial_state is None else initial_state.float()
    outs = []
    for i in range(n):
        Kd, Qd = K[:, :, i] * Dt[:, :, i], Q[:, :, i] * Dt[:, :, i]             # decayed from the chunk start
        rhs = V[:, :, i] - Kd @ S
        R = torch.linalg.solve_triangular(eye + A[:, :, i], rhs, upper=False, unitriangular=True)
        outs.append(Qd @ S + P[:, :, i] @ R)
        Kend = K[:, :, i] * Dend[:, :, i] * Bt[:, :, i].unsqueeze(-1)
        S = S * Dt[:, :, i, -1].unsqueeze(-1) + Kend.transpose(-1, -2) @ R
    o = torch.stack(outs, dim=2)                                                # [B, H, n, C, Dv]
    o = o.permute(0, 2, 3, 1, 4).reshape(B, n * C, H, Dv)[:, :T].to(v.dtype)
    return (o, S) if return_state else o


def _cuda_forward(q, k, v, g, beta):
    from . import _lib
    B, T, H, Dk = q.shape
    Dv = v.size(-1)
    qb, kb, vb = (t.to(torch.bfloat16).contiguous() for t in (q, k, v))
    gf, bf = g.float().contiguous(), beta.float().contiguous()
    o = torch.empty((B, T, H, Dv), dtype=torch.bfloat16, device=q.device)
    P, I = _lib.c_void_p, _lib.c_int
    rc = _lib.fn("sr_gated_delta_fwd", [P] * 7 + [I] * 7 + [P])(
        qb.data_ptr(), kb.data_ptr(), vb.data_ptr(), gf.data_ptr(), bf.data_ptr(), o.data_ptr(), 0, B, T, H, Dk, Dv,
        int(g.dim() == 4), 0, _lib.stream_ptr())
    _lib.check_rc(rc, "sr_gated_delta_fwd")
    return o.to(v.dtype)


def cuda_kernel_usable(q, v) -> bool:
    return q.is_cuda and q.size(-1) in (64, 128) and v.size(-1) >= 1


class _GatedDeltaRuleFn(Function):
    @staticmethod
    def forward(ctx, q, k, v, g, beta):
        ctx.save_for_backward(q, k, v, g, beta)
        return _cuda_forward(q, k, v, g, beta)

    @staticmethod
    def backward(ctx, do):
        saved = ctx.saved_tensors
        with torch.enable_grad():
            ins = [t.detach().requires_grad_(True) for t in saved]
            o = gated_delta_rule_chunked(*ins)
            grads = torch.autograd.grad(o, ins, do.to(o.dtype))
        return tuple(gr.to(t.dtype) for gr, t in zip(grads, saved))


def gated_delta_rule(q, k, v, g, beta, impl="auto"):
    """The op. impl: "auto" (CUDA kernel forward where possible), "chunk", "recurrent" (the oracle, slow)."""
    if impl == "recurrent":
        return gated_delta_rule_recurrent(q, k, v, g, beta)
    if impl == "auto" and cuda_kernel_usable(q, v):
        if torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v, g, beta)):
            return _GatedDeltaRuleFn.apply(q, k, v, g, beta)
        return _cuda_forward(q, k, v, g, beta)
    return gated_delta_rule_chunked(q, k, v, g, beta)
