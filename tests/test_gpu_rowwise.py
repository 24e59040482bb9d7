"""GPU numerics of the fused row-wise kernels of the transformer block, one kernel at a time, each against a plain
fp32 PyTorch statement of the same op (autograd supplies the oracle's backward). Ragged row counts, dropout with
p > 0 (the mask is recovered from the forward output and must be the one the backward uses), both values of the
stochastic-depth keep flag, the key offset and exclusive self-attention variants."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

P, I, L, F32, ULL = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float, ctypes.c_ulonglong
EPS = 0.0078125


def _bf(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).bfloat16()


def _call(name, argtypes, *args):
    from slowrun_b200.ops import _lib
    rc = _lib.fn(name, argtypes)(*args)
    assert rc == 0, (name, rc)


def _sp():
    return torch.cuda.current_stream().cuda_stream


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


def _rms(x):
    return x * torch.rsqrt(x.square().mean(-1, keepdim=True) + EPS)


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def _state():
    from slowrun_b200.ops import functional as ops
    return ops.dropout_state("cuda")


@pytest.mark.parametrize("rows,D,with_skip", [(37, 256, True), (130, 512, False), (8, 2560, True)])
def test_mix_norm_forward_and_backward(rows, D, with_skip):
    xp, x0 = _bf(rows, D, seed=1), _bf(rows, D, seed=2)
    sk = _bf(rows, D, seed=3) if with_skip else None
    scal = torch.tensor([1.1, 0.2, 0.7], device="cuda")
    x, a = torch.empty_like(xp), torch.empty_like(xp)
    _call("sr_mix_norm_fwd", [P] * 8 + [L, I, F32, P], xp.data_ptr(), x0.data_ptr(), _ptr(sk), x.data_ptr(), a.data_ptr(),
          scal.data_ptr(), scal.data_ptr() + 4, scal.data_ptr() + 8 if with_skip else 0, rows, D, EPS, _sp())
    # oracle
    xpf, x0f = xp.float().requires_grad_(True), x0.float().requires_grad_(True)
    skf = sk.float().requires_grad_(True) if with_skip else None
    sc = scal.clone().requires_grad_(True)
    xr = sc[0] * (xpf + (sc[2] * skf if with_skip else 0)) + sc[1] * x0f
    ar = _rms(xr)
    assert _rel(x, xr) < 6e-3 and _rel(a, ar) < 8e-3
    # backward: gradients of (a, x) -> inputs, with a second residual gradient as the stochastic-depth bypass adds it
    da, g_res, g_res2 = _bf(rows, D, seed=4), _bf(rows, D, seed=5), _bf(rows, D, seed=6)
    (ar * da.float()).sum().backward(retain_graph=True)
    (xr * (g_res.float() + g_res2.float())).sum().backward()
    dxp, dx0 = torch.empty_like(xp), torch.empty_like(xp)
    dsk = torch.empty_like(xp) if with_skip else None
    dscal = torch.zeros(3, device="cuda")
    _call("sr_norm_bwd_mix", [P] * 16 + [L, I, F32, P], x.data_ptr(), da.data_ptr(), g_res.data_ptr(), g_res2.data_ptr(),
          xp.data_ptr(), x0.data_ptr(), _ptr(sk), dxp.data_ptr(), dx0.data_ptr(), _ptr(dsk), scal.data_ptr(),
          scal.data_ptr() + 4, scal.data_ptr() + 8 if with_skip else 0, dscal.data_ptr(), dscal.data_ptr() + 4,
          dscal.data_ptr() + 8 if with_skip else 0, rows, D, EPS, _sp())
    torch.cuda.synchronize()
    assert _rel(dxp, xpf.grad) < 1.2e-2 and _rel(dx0, x0f.grad) < 1.2e-2
    if with_skip:
        assert _rel(dsk, skf.grad) < 1.2e-2
    want = sc.grad if with_skip else sc.grad[:2]
    got = dscal if with_skip else dscal[:2]
    assert torch.allclose(got, want, rtol=3e-2, atol=3e-2 * want.abs().max().item()), (got, want)


@pytest.mark.parametrize("rows,D,p", [(37, 256, 0.0), (130, 512, 0.25), (9, 2560, 0.1)])
def test_add_norm_forward_and_norm_bwd_drop_share_one_mask(rows, D, p):
    x = _bf(rows, D, seed=7)
    y = (_bf(rows, D, seed=8).float().abs() + 1.0).bfloat16()               # bounded away from 0: the mask is recoverable
    seed = 0x1234567
    x_mid, n = torch.empty_like(x), torch.empty_like(x)
    _call("sr_add_norm_fwd", [P] * 4 + [L, I, F32, F32, ULL, P, P], x.data_ptr(), y.data_ptr(), x_mid.data_ptr(), n.data_ptr(),
          rows, D, EPS, p, seed, _state().data_ptr(), _sp())
    branch = x_mid.float() - x.float()
    mask = (branch.abs() > 0.25 * y.float().abs()).float()                  # kept elements carry y / (1 - p)
    if p == 0.0:
        assert mask.min().item() == 1.0
    else:
        assert abs(mask.mean().item() - (1 - p)) < 0.03
    xr = x.float().requires_grad_(True)
    yr = y.float().requires_grad_(True)
    xm = xr + yr * mask / (1 - p)
    nr = _rms(xm)
    assert _rel(x_mid, xm) < 6e-3 and _rel(n, nr) < 8e-3
    dn, g_res = _bf(rows, D, seed=9), _bf(rows, D, seed=10)
    (nr * dn.float()).sum().backward(retain_graph=True)
    (xm * g_res.float()).sum().backward()
    dx_mid, dy = torch.empty_like(x), torch.empty_like(x)
    _call("sr_norm_bwd_drop", [P] * 5 + [L, I, F32, F32, ULL, P, P], x_mid.data_ptr(), dn.data_ptr(), g_res.data_ptr(),
          dx_mid.data_ptr(), dy.data_ptr(), rows, D, EPS, p, seed, _state().data_ptr(), _sp())
    torch.cuda.synchronize()
    assert _rel(dx_mid, xr.grad) < 1.2e-2
    assert _rel(dy, yr.grad) < 1.2e-2
    # exactly the dropped positions of the forward carry no gradient in the backward
    assert torch.equal(dy.float() == 0, (mask == 0) | (dx_mid.float() == 0))


@pytest.mark.parametrize("keep", [0.0, 1.0])
@pytest.mark.parametrize("p", [0.0, 0.2])
def test_dropout_add_with_stochastic_depth_keep_flag(keep, p):
    n = 64 * 520
    x_mid, y, x_in = _bf(n, seed=11), (_bf(n, seed=12).float().abs() + 1.0).bfloat16(), _bf(n, seed=13)
    kt = torch.full((), keep, device="cuda")
    out = torch.empty_like(x_mid)
    seed = 0x7654321
    _call("sr_dropout_add_fwd", [P] * 5 + [L, F32, ULL, P, P], x_mid.data_ptr(), y.data_ptr(), x_in.data_ptr(), kt.data_ptr(),
          out.data_ptr(), n, p, seed, _state().data_ptr(), _sp())
    if keep == 0.0:
        assert torch.equal(out, x_in)
    g = _bf(n, seed=14)
    dy, dmid, din = torch.empty_like(g), torch.empty_like(g), torch.empty_like(g)
    _call("sr_dropout_add_bwd", [P] * 5 + [L, F32, ULL, P, P], g.data_ptr(), kt.data_ptr(), dy.data_ptr(), dmid.data_ptr(),
          din.data_ptr(), n, p, seed, _state().data_ptr(), _sp())
    torch.cuda.synchronize()
    if keep == 0.0:
        assert dy.abs().max().item() == 0 and dmid.abs().max().item() == 0 and torch.equal(din, g)
    else:
        mask = ((out.float() - x_mid.float()).abs() > 0.25 * y.float().abs()).float()
        assert _rel(out, x_mid.float() + y.float() * mask / (1 - p)) < 6e-3
        assert _rel(dy, g.float() * mask / (1 - p)) < 6e-3
        assert torch.equal(dmid, g) and din.abs().max().item() == 0


def _rope_norm(x, cos, sin):
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    return _rms(torch.cat([x1 * cos + x2 * sin, -x1 * sin + x2 * cos], -1))


@pytest.mark.parametrize("B,T,H,key_offset,with_ve", [(2, 37, 3, False, True), (1, 64, 2, True, False), (3, 19, 2, True, True)])
@pytest.mark.parametrize("f32dq", [False, True])
def test_qkv_prep_forward_and_backward(B, T, H, key_offset, with_ve, f32dq):
    D, M = 128, B * T
    C = H * D
    qkv = _bf(M, 3 * C, seed=20)
    ve = _bf(M, C, seed=21) if with_ve else None
    gate = (torch.rand(M, H, device="cuda", generator=torch.Generator(device="cuda").manual_seed(22)) * 2) if with_ve else None
    ang = torch.rand(T, 64, device="cuda", generator=torch.Generator(device="cuda").manual_seed(23)) * 6.28
    cos, sin = ang.cos().bfloat16(), ang.sin().bfloat16()
    q, k, v = (torch.empty(B, T, H, D, dtype=torch.bfloat16, device="cuda") for _ in range(3))
    _call("sr_qkv_prep_fwd", [P] * 8 + [L, I, I, F32, I, P], qkv.data_ptr(), _ptr(ve), _ptr(gate), cos.data_ptr(), sin.data_ptr(),
          q.data_ptr(), k.data_ptr(), v.data_ptr(), M, H, T, EPS, int(key_offset), _sp())
    # oracle
    qr = qkv.float().requires_grad_(True)
    ver = ve.float().requires_grad_(True) if with_ve else None
    gr = gate.clone().requires_grad_(True) if with_ve else None
    x = qr.view(B, T, 3, H, D)
    c4, s4 = cos.float().view(1, T, 1, 64), sin.float().view(1, T, 1, 64)
    q_o, k_o = _rope_norm(x[:, :, 0], c4, s4), _rope_norm(x[:, :, 1], c4, s4)
    if key_offset and T > 1:
        k_o = torch.cat([k_o[..., :64], torch.cat([k_o[:, :1, :, 64:], k_o[:, :-1, :, 64:]], 1)], -1)
    v_o = x[:, :, 2]
    if with_ve:
        v_o = v_o + gr.view(B, T, H, 1) * ver.view(B, T, H, D)
    assert _rel(q, q_o) < 8e-3 and _rel(k, k_o) < 8e-3 and _rel(v, v_o) < 8e-3
    dq, dk, dv = _bf(B, T, H, D, seed=24), _bf(B, T, H, D, seed=25), _bf(B, T, H, D, seed=26)
    dvx = _bf(B, T, H, D, seed=27)
    ((q_o * dq.float()).sum() + (k_o * dk.float()).sum() + (v_o * (dv.float() + dvx.float())).sum()).backward()
    dqkv = torch.empty_like(qkv)
    dve = torch.empty_like(ve) if with_ve else None
    dgate = torch.empty_like(gate) if with_ve else None
    dq_arg = dq.float().contiguous() if f32dq else dq
    _call("sr_qkv_prep_bwd_f32dq" if f32dq else "sr_qkv_prep_bwd", [P] * 11 + [L, I, I, F32, I, P, P], qkv.data_ptr(), _ptr(ve),
          _ptr(gate), cos.data_ptr(), sin.data_ptr(), dq_arg.data_ptr(), dk.data_ptr(), dv.data_ptr(), dqkv.data_ptr(),
          _ptr(dve), _ptr(dgate), M, H, T, EPS, int(key_offset), dvx.data_ptr(), _sp())
    torch.cuda.synchronize()
    assert _rel(dqkv, qr.grad) < 1.2e-2, _rel(dqkv, qr.grad)
    if with_ve:
        assert _rel(dve, ver.grad) < 1.2e-2
        assert _rel(dgate, gr.grad) < 1.2e-2


@pytest.mark.parametrize("B,T,H,xsa", [(2, 37, 3, False), (2, 37, 3, True), (1, 130, 8, True)])
def test_attn_post_forward_and_backward(B, T, H, xsa):
    D, M = 128, B * T
    y, v = _bf(B, T, H, D, seed=30), _bf(B, T, H, D, scale=0.5, seed=31)
    if xsa:
        v[0, 1, 0] *= 1e-5       # a norm below the clamp: v^ = v / eps there
    gate = torch.rand(M, H, device="cuda", generator=torch.Generator(device="cuda").manual_seed(32))
    alpha = torch.tensor([0.3 * (i - H / 2) for i in range(H)], device="cuda") if xsa else None
    eps_x = 1e-4
    out = torch.empty_like(y)
    _call("sr_attn_post_fwd", [P] * 5 + [L, I, F32, P], y.data_ptr(), v.data_ptr(), gate.data_ptr(), _ptr(alpha), out.data_ptr(),
          M, H, eps_x, _sp())
    yr, vr = y.float().requires_grad_(True), v.float().requires_grad_(True)
    gr = gate.clone().requires_grad_(True)
    ar = alpha.clone().requires_grad_(True) if xsa else None
    yy = yr
    if xsa:
        vh = vr / vr.square().sum(-1, keepdim=True).sqrt().clamp_min(eps_x)
        yy = yr - torch.tanh(ar).view(1, 1, H, 1) * (yr * vh).sum(-1, keepdim=True) * vh
    o_r = yy * gr.view(B, T, H, 1)
    assert _rel(out, o_r) < 6e-3
    g = _bf(B, T, H, D, seed=33)
    (o_r * g.float()).sum().backward()
    dy = torch.empty_like(y)
    dgate = torch.empty_like(gate)
    delta = torch.empty(B, H, T, device="cuda")
    dvx = torch.empty_like(y) if xsa else None
    dalpha = torch.full((H,), 0.5, device="cuda") if xsa else None       # accumulated into: starts non-zero
    _call("sr_attn_post_bwd", [P] * 10 + [L, I, I, F32, P], g.data_ptr(), y.data_ptr(), v.data_ptr(), gate.data_ptr(), _ptr(alpha),
          dy.data_ptr(), dgate.data_ptr(), delta.data_ptr(), _ptr(dvx), _ptr(dalpha), M, H, T, eps_x, _sp())
    torch.cuda.synchronize()
    assert _rel(dy, yr.grad) < 8e-3
    assert _rel(dgate, gr.grad) < 8e-3
    want_delta = (yr.grad * y.float()).sum(-1).permute(0, 2, 1)
    assert _rel(delta, want_delta) < 1e-2
    if xsa:
        keep = torch.ones(B, T, H, 1, device="cuda")
        keep[0, 1, 0] = 0                  # the clamped row: its dv has a 1/eps factor, compare it separately
        assert _rel(dvx.float() * keep, vr.grad * keep) < 1.2e-2
        assert _rel(dvx[0, 1, 0], vr.grad[0, 1, 0]) < 2e-2
        assert torch.allclose(dalpha - 0.5, ar.grad, rtol=2e-2, atol=2e-2 * ar.grad.abs().max().item())


def test_dropout_masks_have_the_right_statistics_and_never_repeat():
    """What the reference gets from torch's Philox dropout (train.py:301, 322: F.dropout) and its per-block
    `torch.rand(())` stochastic depth (train.py:338-341), checked as statistics since the streams differ by construction:
    keep rate within four standard errors of 1 - p, no correlation between neighbouring elements or rows, a fresh mask
    for every call site (salt) and every step (device counter), and the same mask again only for the same (site, step)."""
    from slowrun_b200.ops import functional as ops
    rows, D, p = 4096, 1024, 0.1
    x = torch.zeros(rows, D, device="cuda", dtype=torch.bfloat16)
    y = torch.ones(rows, D, device="cuda", dtype=torch.bfloat16)
    st = ops.dropout_state("cuda")
    st.fill_(0x1234ABCD5)            # a fixed step counter: the checks below are then the same numbers on every run

    def mask(seed):
        out = torch.empty_like(x)
        _call("sr_dropout_add_fwd", [P] * 5 + [L, F32, ULL, P, P], x.data_ptr(), y.data_ptr(), 0, 0, out.data_ptr(), x.numel(), p,
              seed, st.data_ptr(), _sp())
        return (out.float() != 0)

    m1 = mask(0x1111)
    n = m1.numel()
    se = (p * (1 - p) / n) ** 0.5
    assert abs(m1.float().mean().item() - (1 - p)) < 4 * se
    # kept values are scaled by 1 / (1 - p)
    out_val = 1.0 / (1 - p)
    f = m1.float()
    # neighbours along the row and along the column are uncorrelated (|r| below 4 / sqrt(n))
    for a, b in ((f[:, 1:], f[:, :-1]), (f[1:], f[:-1])):
        r = torch.corrcoef(torch.stack([a.reshape(-1), b.reshape(-1)]))[0, 1].item()
        assert abs(r) < 4 / n ** 0.5, r
    # per-row and per-column keep rates show no stripe
    assert (f.mean(1) - (1 - p)).abs().max().item() < 6 * (p * (1 - p) / D) ** 0.5
    assert (f.mean(0) - (1 - p)).abs().max().item() < 6 * (p * (1 - p) / rows) ** 0.5
    # another call site: an independent mask (agreement rate = p^2 + (1-p)^2 within 4 standard errors)
    m2 = mask(0x2222)
    agree = (m1 == m2).float().mean().item()
    q = p * p + (1 - p) * (1 - p)
    assert abs(agree - q) < 4 * (q * (1 - q) / n) ** 0.5, agree
    # same site, same step: the same mask (what the backward pass relies on); next step: a fresh one
    assert torch.equal(mask(0x1111), m1)
    ops.advance_dropout_state("cuda")
    m3 = mask(0x1111)
    agree = (m1 == m3).float().mean().item()
    assert abs(agree - q) < 4 * (q * (1 - q) / n) ** 0.5, agree
    assert out_val > 1.0


def test_stochastic_depth_keep_rate():
    """Block i is skipped with probability stoch_depth * i / (n_layer - 1) (train.py:332-341); the keep flags the block
    node draws follow that rate."""
    from slowrun_b200.config import track_defaults
    from slowrun_b200.models.gpt import build_model
    cfg = track_defaults("limited")
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len, m.stoch_depth = 4, 256, 2, 2, 128, 0.5
    model = build_model(m, "cuda", seed=0)
    probs = [blk.drop_prob for blk in model.transformer.h]
    assert probs == pytest.approx([0.5 * i / 3 for i in range(4)])
    torch.manual_seed(0)
    draws = torch.rand(4000, device="cuda")
    for pr in probs[1:]:
        keep = (draws >= pr).float().mean().item()
        assert abs(keep - (1 - pr)) < 4 * (pr * (1 - pr) / 4000) ** 0.5
