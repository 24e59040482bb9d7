"""GPU numerics of the fused lm-head + soft-capped cross-entropy kernels and of the fp8 GEMM they build on, each
against a plain-PyTorch fp32 statement of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _bf(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).bfloat16()


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


def _status_ok():
    from slowrun_b200.ops import _lib
    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (300, 520, 272), (1000, 1288, 2560), (256, 128, 4096)])
@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
def test_gemm_fp8_matches_fp32_product_of_the_quantised_operands(M, N, K, fmt):
    from slowrun_b200.ops.gemm import gemm_fp8, quantize_fp8
    dt = torch.float8_e4m3fn if fmt == "e4m3" else torch.float8_e5m2
    a, b = _bf(M, K, seed=1), _bf(N, K, scale=0.5, seed=2)
    sa, sb = 4.0 / 448, 2.0 / 448
    qa, qb = quantize_fp8(a, sa, dtype=dt), quantize_fp8(b, sb)
    # the quantiser itself: same values as torch's saturating cast of the scaled tensor
    want_a = (a.float() / sa).clamp(-torch.finfo(dt).max, torch.finfo(dt).max).to(dt)
    assert (qa.float() - want_a.float()).abs().max().item() <= 0.13 * want_a.float().abs().max().item()
    assert _rel(qa.float(), want_a.float()) < 2e-2
    out = gemm_fp8(qa, qb, alpha=sa * sb, out_dtype=torch.float32)
    ref = (qa.float() @ qb.float().t()) * (sa * sb)
    _status_ok()
    assert _rel(out, ref) < 2e-3, _rel(out, ref)
    # and the quantised product tracks the unquantised one to fp8 accuracy
    assert _rel(out, a.float() @ b.float().t()) < 0.12


def test_quantize_fp8_transposed_layout():
    from slowrun_b200.ops.gemm import quantize_fp8
    x = _bf(200, 328, seed=3)
    q = quantize_fp8(x, 0.01)
    qt = quantize_fp8(x, 0.01, transpose=True)
    assert qt.shape == (328, 200)
    assert torch.equal(qt.float(), q.float().t())


def _oracle(x, w, w_t, tgt, cap, vocab, weights):
    from slowrun_b200.ops import functional as ops
    xb = x.float().clone().requires_grad_(True)
    wb = w.float().clone().requires_grad_(True)
    logits = (xb @ wb) if w_t else (xb @ wb.t())
    loss = ops.softcap_ce_ref(logits, tgt, cap, vocab, weights)
    return xb, wb, logits, loss


@pytest.mark.parametrize("M,d,V,Vpad", [(300, 256, 1000, 1024), (1100, 512, 1500, 1536), (513, 320, 50257, 50304)])
@pytest.mark.parametrize("weights", [None, [1.0, 0.5, 0.25]])
@pytest.mark.parametrize("w_t", [False, True])
def test_fused_head_matches_oracle_and_the_unfused_path(M, d, V, Vpad, weights, w_t):
    from slowrun_b200.ops import functional as ops
    x = _bf(M, d, seed=16)
    w = _bf(d, Vpad, scale=0.08, seed=17) if w_t else _bf(Vpad, d, scale=0.08, seed=17)
    tgt = torch.randint(0, V, (M,), device="cuda")
    if weights is None:
        tgt[:7] = -1
        tgt[-1] = -1
    else:
        tgt[10:14] = 5          # equal targets inside one row's window
    wt = None if weights is None else torch.tensor(weights, device="cuda")
    vocab = V if weights is None else Vpad
    res = {}
    for fused in (True, False):
        ops.set_fused_head(fused)
        try:
            xa = x.clone().requires_grad_(True)
            acc = torch.zeros(w.shape, dtype=torch.float32, device="cuda")
            loss = ops.lm_head_loss(xa, w, tgt, 15.0, vocab, grad_acc=acc, w_t=w_t, weights=wt)
            (loss * 0.5).backward()
            rows = ops.lm_head_rows(x, w, tgt, 15.0, V, w_t=w_t)
            res[fused] = (loss.item(), xa.grad.clone(), acc, rows)
        finally:
            ops.set_fused_head(True)
    xb, wb, logits, lref = _oracle(x, w, w_t, tgt, 15.0, vocab, wt)
    (lref * 0.5).backward()
    rref = ops.softcap_ce_ref(logits.detach(), tgt, 15.0, V, None, "none")
    _status_ok()
    loss, dx, dw, rows = res[True]
    assert abs(loss - lref.item()) < 2e-3 * abs(lref.item()), (loss, lref.item())
    assert _rel(dx, xb.grad) < 1.5e-2, _rel(dx, xb.grad)
    assert _rel(dw, wb.grad) < 1.5e-2, _rel(dw, wb.grad)
    assert _rel(rows, rref) < 2e-3
    # ignored rows carry no gradient
    if weights is None:
        assert dx[:7].abs().max().item() == 0.0
    # the fused path is at least as close to the oracle as the logits-through-memory path
    assert _rel(dx, xb.grad) <= 1.5 * _rel(res[False][1], xb.grad) + 1e-3
    assert abs(loss - lref.item()) <= abs(res[False][0] - lref.item()) + 1e-3 * abs(lref.item())


@pytest.mark.parametrize("M,w_t", [(700, True), (1024, False)])
def test_fused_head_fp8_tracks_the_quantised_oracle(M, w_t):
    """Forward against the oracle evaluated on the operands as the kernel sees them (e4m3 values times the static
    scales); backward (e5m2 gradient, e4m3 x and W, fp32 accumulation) against the fp32 gradients to fp8 accuracy."""
    from slowrun_b200.ops import functional as ops
    d, Vpad = 512, 1536
    x = _bf(M, d, seed=21)
    w = _bf(d, Vpad, scale=0.004, seed=22) if w_t else _bf(Vpad, d, scale=0.004, seed=22)   # [d, V] as in the tiny track
    tgt = torch.randint(0, Vpad, (M,), device="cuda")
    wt = torch.tensor([1.0, 0.5, 0.25], device="cuda")
    xa = x.clone().requires_grad_(True)
    acc = torch.zeros(w.shape, dtype=torch.float32, device="cuda")
    loss = ops.lm_head_loss(xa, w, tgt, 15.0, Vpad, grad_acc=acc, w_t=w_t, weights=wt, fp8=True)
    (loss * 0.5).backward()
    # oracle on the operands as the kernel sees them: e4m3 values times the static scales
    xq = (x.float() / ops.FP8_X_SCALE).clamp(-448, 448).to(torch.float8_e4m3fn).float() * ops.FP8_X_SCALE
    wq = (w.float() / ops.FP8_W_SCALE).clamp(-448, 448).to(torch.float8_e4m3fn).float() * ops.FP8_W_SCALE
    lq = ops.softcap_ce_ref((xq @ wq) if w_t else (xq @ wq.t()), tgt, 15.0, Vpad, wt)
    xb, wb, _, lref = _oracle(x, w, w_t, tgt, 15.0, Vpad, wt)
    (lref * 0.5).backward()
    _status_ok()
    assert abs(loss.item() - lq.item()) < 2e-3 * abs(lq.item()), (loss.item(), lq.item())
    assert abs(loss.item() - lref.item()) < 2e-2 * abs(lref.item())
    assert _rel(xa.grad, xb.grad) < 0.15, _rel(xa.grad, xb.grad)
    assert _rel(acc, wb.grad) < 0.15, _rel(acc, wb.grad)
