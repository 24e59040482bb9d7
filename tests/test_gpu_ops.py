"""GPU numerics: every CUDA kernel against the plain-PyTorch fp32 statement of the same op (forward and backward)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _bf(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).bfloat16()


def _close(a, b, rtol=2e-2, atol=2e-2, rel=1.5e-2):
    """Largest error against the largest reference magnitude (catches a single wrong element) and the relative Frobenius
    error (catches a systematic few-percent error that the first bound would let through); `rel` is 1.5e-2 for bf16
    results and is passed smaller for fp32 ones."""
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item()
    assert err <= atol * max(ref, 1e-6) + rtol * 1e-3 or torch.allclose(a, b, rtol=rtol, atol=atol * max(ref, 1e-3)), (err, ref)
    fro = ((a - b).norm() / b.norm().clamp_min(1e-20)).item()
    assert fro <= rel, ("relative Frobenius error", fro)


def _status_ok():
    from slowrun_b200.ops import _lib
    torch.cuda.synchronize()
    _lib.check_status()


# ------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("M,N,K,batch,a_mn,b_mn,bn", [
    (128, 256, 64, 1, False, False, 256), (128, 128, 128, 1, False, False, 128), (512, 768, 320, 1, False, False, 0),
    (200, 328, 136, 2, False, False, 0), (256, 512, 256, 1, False, True, 0), (256, 512, 256, 1, True, True, 0),
    (256, 512, 256, 1, True, False, 0), (8188, 2560, 512, 1, False, False, 0), (20, 4096, 24, 3, False, False, 0),
    (1024, 2560, 320, 1, False, False, 160), (640, 480, 256, 2, False, True, 160), (384, 320, 192, 1, True, True, 160),
])
def test_gemm_modes(M, N, K, batch, a_mn, b_mn, bn):
    from slowrun_b200.ops.gemm import gemm, gemm_reference
    A = _bf(batch, *((K, M) if a_mn else (M, K)), scale=0.1, seed=1)
    B = _bf(batch, *((K, N) if b_mn else (N, K)), scale=0.1, seed=2)
    out = gemm(A, B, a_mn=a_mn, b_mn=b_mn, alpha=1.5, bn=bn)
    ref = gemm_reference(A, B, a_mn=a_mn, b_mn=b_mn, alpha=1.5, out_dtype=torch.float32)
    _status_ok()
    _close(out, ref)


@pytest.mark.parametrize("K,Mo,No,bn", [(1024, 384, 640, 0), (8192, 2560, 2560, 0), (4100 // 4 * 4, 200, 328, 0), (1024, 384, 640, -256)])
def test_gemm_fp32_accumulate_and_device_alpha(K, Mo, No, bn):
    """dW[Mo, No] += alpha * A^T B with the k-loop balanced over all SMs (bn < 0 forces the plain tile schedule)."""
    from slowrun_b200.ops.gemm import gemm, gemm_reference
    A, B = _bf(K, Mo, scale=0.1, seed=1), _bf(K, No, scale=0.1, seed=2)
    acc = torch.randn(Mo, No, device="cuda")
    ref = gemm_reference(A, B, acc.clone(), a_mn=True, b_mn=True, alpha=0.25, beta=1.0, out_dtype=torch.float32)
    gemm(A, B, out=acc, cin=acc, a_mn=True, b_mn=True, beta=1.0, alpha_t=torch.tensor(0.25, device="cuda"), bn=bn)
    _status_ok()
    assert torch.allclose(acc, ref, rtol=2e-3, atol=2e-3 * ref.abs().max().item())


@pytest.mark.parametrize("pair", [True, False])
@pytest.mark.parametrize("M,N,K,a_mn,b_mn,bn", [
    (8192, 2560, 320, False, True, 256),    # 320 pair tiles: 4 full waves + a column-sliced tail
    (8192, 2500, 264, False, False, 256),   # same with a ragged right edge inside the sliced tiles
    (512, 512, 512, False, False, 256),     # fewer tiles than CTA pairs
    (2048, 1280, 512, True, False, 160), (1024, 896, 384, True, True, 128), (300, 200, 136, False, True, 0),
])
def test_gemm_pair_and_single_cta_kernels(pair, M, N, K, a_mn, b_mn, bn):
    """The CTA-pair kernel (default) and the single-CTA kernel give the same product on every operand layout."""
    from slowrun_b200.ops.gemm import gemm, gemm_reference, set_pair_mode
    A = _bf(*((K, M) if a_mn else (M, K)), scale=0.1, seed=5)
    B = _bf(*((K, N) if b_mn else (N, K)), scale=0.1, seed=6)
    set_pair_mode(pair)
    try:
        out = gemm(A, B, a_mn=a_mn, b_mn=b_mn, bn=bn)
    finally:
        set_pair_mode(True)
    _status_ok()
    _close(out, gemm_reference(A, B, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32))


@pytest.mark.parametrize("n,g,k,bn", [(3, 768, 512, 0), (2, 640, 256, 128), (1, 2560, 1024, 0), (2, 904, 264, 0), (1, 1288, 320, 256)])
def test_gemm_symmetric(n, g, k, bn):
    from slowrun_b200.ops.gemm import gemm, gemm_reference
    X = _bf(n, g, k, scale=0.05, seed=3)
    S = _bf(n, g, g, scale=0.5, seed=4)
    S = (S + S.transpose(1, 2)).contiguous()
    out = gemm(X, X, cin=S, alpha=2.0, beta=0.5, sym=True, bn=bn)
    ref = gemm_reference(X, X, S, alpha=2.0, beta=0.5, out_dtype=torch.float32)
    _status_ok()
    _close(out, ref)
    assert torch.equal(out, out.transpose(1, 2)), "mirrored store must give an exactly symmetric result"


# ------------------------------------------------------------------ elementwise family
def _check_fwd_bwd(fn_cuda, fn_ref, inputs, grad_inputs, rtol=3e-2, atol=3e-2):
    """inputs: list of bf16 CUDA tensors; grad_inputs: indices that need gradients."""
    a = [t.detach().clone().requires_grad_(i in grad_inputs) for i, t in enumerate(inputs)]
    b = [t.detach().float().clone().requires_grad_(i in grad_inputs) for i, t in enumerate(inputs)]
    ya, yb = fn_cuda(*a), fn_ref(*b)
    _close(ya, yb, rtol, atol)
    g = torch.randn_like(yb)
    ya.backward(g.to(ya.dtype))
    yb.backward(g)
    _status_ok()
    for i in grad_inputs:
        _close(a[i].grad, b[i].grad, rtol, atol)


def test_rmsnorm():
    from slowrun_b200.ops import functional as ops
    x = _bf(4, 300, 2560, seed=5)
    _check_fwd_bwd(lambda t: ops.rms_norm(t, 1e-6), lambda t: ops.rms_norm_ref(t, 1e-6), [x], [0])


def test_swiglu():
    from slowrun_b200.ops import functional as ops
    gf = _bf(3, 200, 2 * 1024, seed=6)
    _check_fwd_bwd(ops.swiglu, ops.swiglu_ref, [gf], [0])


def test_rope_qknorm_on_strided_view():
    from slowrun_b200.ops import functional as ops
    B, T, H, D = 2, 96, 3, 128
    qkv = _bf(B, T, 3 * H * D, seed=7)
    t = torch.arange(T, device="cuda").float()
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    fr = torch.outer(t, inv)
    cos, sin = fr.cos().bfloat16()[None, :, None, :], fr.sin().bfloat16()[None, :, None, :]

    def cuda_fn(x):
        return ops.rope_qknorm(x.view(B, T, 3, H, D)[:, :, 1], cos, sin, 1e-6)

    def ref_fn(x):
        return ops.rope_qknorm_ref(x.view(B, T, 3, H, D)[:, :, 1], cos.float(), sin.float(), 1e-6)
    _check_fwd_bwd(cuda_fn, ref_fn, [qkv], [0])


def test_head_gates():
    from slowrun_b200.ops import functional as ops
    B, T, H, D = 2, 64, 5, 128
    v, ve = _bf(B, T, H, D, seed=8), _bf(B, T, H, D, seed=9)
    gate = torch.rand(B, T, H, device="cuda").bfloat16()
    _check_fwd_bwd(ops.gated_add, ops.gated_add_ref, [v, gate, ve], [0, 1, 2])
    _check_fwd_bwd(ops.head_scale, ops.head_scale_ref, [v, gate], [0, 1])


def test_lambda_mix_accumulates_scalar_grads():
    from slowrun_b200.ops import functional as ops
    x, x0, sk = _bf(2, 64, 512, seed=10), _bf(2, 64, 512, seed=11), _bf(2, 64, 512, seed=12)
    lr = torch.nn.Parameter(torch.tensor([0.9, 1.1], device="cuda"))
    l0 = torch.nn.Parameter(torch.tensor([0.1, 0.2], device="cuda"))
    ws = torch.nn.Parameter(torch.tensor([0.7], device="cuda"))
    xa, x0a, ska = (t.clone().requires_grad_(True) for t in (x, x0, sk))
    y = ops.lambda_mix(xa, x0a, ska, lr, l0, ws, 1, 0)
    g = torch.randn_like(y.float())
    y.backward(g.bfloat16())
    xb, x0b, skb = (t.float().clone().requires_grad_(True) for t in (x, x0, sk))
    lrb, l0b, wsb = (p.detach().clone().requires_grad_(True) for p in (lr, l0, ws))
    yb = ops.lambda_mix_ref(xb, x0b, skb, lrb[1], l0b[1], wsb[0])
    yb.backward(g.bfloat16().float())
    _status_ok()
    _close(y, yb)
    for a, b in ((xa.grad, xb.grad), (x0a.grad, x0b.grad), (ska.grad, skb.grad)):
        _close(a, b)
    assert torch.allclose(lr.grad, lrb.grad, rtol=2e-2, atol=1e-1)
    assert torch.allclose(l0.grad, l0b.grad, rtol=2e-2, atol=1e-1)
    assert torch.allclose(ws.grad, wsb.grad, rtol=2e-2, atol=1e-1)


def test_dropout_add_mask_is_reproduced_in_backward():
    from slowrun_b200.ops import functional as ops
    x, y = _bf(4, 64, 512, seed=13), _bf(4, 64, 512, seed=14)
    xa, ya = x.clone().requires_grad_(True), y.clone().requires_grad_(True)
    torch.manual_seed(3)
    out = ops.dropout_add(xa, ya, 0.25, True)
    out.backward(torch.ones_like(out))
    _status_ok()
    # gradient w.r.t. y is mask/(1-p): zero where dropped, 4/3 where kept
    gy = ya.grad.float()
    kept = gy != 0
    frac = kept.float().mean().item()
    assert 0.70 < frac < 0.80, frac
    assert torch.allclose(gy[kept], torch.full_like(gy[kept], 1 / 0.75), rtol=1e-2)
    # the forward used the same mask: out == x + y/(1-p) where kept, out == x where dropped
    expect = torch.where(kept, x.float() + y.float() / 0.75, x.float())
    _close(out, expect)
    assert torch.equal(out[~kept], x[~kept])
    assert torch.equal(xa.grad, torch.ones_like(xa.grad))
    # stochastic-depth form
    keep = torch.zeros((), device="cuda")
    xin = _bf(4, 64, 512, seed=15)
    assert torch.equal(ops.dropout_add(x, y, 0.0, True, x_in=xin, keep=keep), xin)
    keep = torch.ones((), device="cuda")
    _close(ops.dropout_add(x, y, 0.0, True, x_in=xin, keep=keep), x.float() + y.float())


@pytest.mark.parametrize("weights", [None, [1.0, 0.5, 0.25]])
@pytest.mark.parametrize("w_t", [False, True])
def test_lm_head_loss(weights, w_t):
    from slowrun_b200.ops import functional as ops
    M, d, V, Vpad = 300, 256, 1000, 1024
    x = _bf(M, d, seed=16)
    w = _bf(d, Vpad, scale=0.05, seed=17) if w_t else _bf(Vpad, d, scale=0.05, seed=17)
    tgt = torch.randint(0, V, (M,), device="cuda")
    if weights is None:
        tgt[:7] = -1
    wt = None if weights is None else torch.tensor(weights, device="cuda")
    vocab = V if weights is None else Vpad
    xa = x.clone().requires_grad_(True)
    acc = torch.zeros(w.shape, dtype=torch.float32, device="cuda")
    loss = ops.lm_head_loss(xa, w, tgt, 15.0, vocab, grad_acc=acc, w_t=w_t, weights=wt)
    (loss * 0.5).backward()
    xb = x.float().clone().requires_grad_(True)
    wb = w.float().clone().requires_grad_(True)
    logits = (xb @ wb) if w_t else (xb @ wb.t())
    lref = ops.softcap_ce_ref(logits, tgt, 15.0, vocab, wt)
    (lref * 0.5).backward()
    _status_ok()
    assert abs(loss.item() - lref.item()) < 2e-2 * abs(lref.item()), (loss.item(), lref.item())
    _close(xa.grad, xb.grad, 5e-2, 5e-2)
    _close(acc, wb.grad, 5e-2, 5e-2)
    rows = ops.lm_head_rows(x, w, tgt, 15.0, V, w_t=w_t)
    rref = ops.softcap_ce_ref(logits.detach(), tgt, 15.0, V, None, "none")
    _close(rows, rref, 3e-2, 3e-2)


# ------------------------------------------------------------------ optimizer kernels
@pytest.mark.parametrize("shape", [(3, 256, 256), (2, 512, 128), (2, 128, 640)])
def test_muon_cuda_path_matches_oracle(shape):
    from slowrun_b200.optim.muon_adamw import muon_update_ref, newton_schulz_cuda, newton_schulz_ref, _NSWorkspace
    from slowrun_b200.ops import _lib
    n, r, c = shape
    torch.manual_seed(0)
    k = 4 * max(r, c)
    A = torch.randn(n, r, k, device="cuda") * torch.logspace(0, -1.5, k, device="cuda")
    G = (A @ torch.randn(n, k, c, device="cuda")) * 0.01
    M0 = torch.randn(n, r, c, device="cuda") * 0.01
    # Newton-Schulz alone, from the same bf16 start. Both bf16 implementations are compared with the same iteration
    # carried out in fp32: ours must be as close to it as torch's bf16 matmul path is.
    X0 = (G / G.norm(dim=(-2, -1), keepdim=True) / 1.02).bfloat16()
    ws = _NSWorkspace(n, r, c, "cuda")
    ours = newton_schulz_cuda(X0.clone(), 5, ws).float()
    ref16 = newton_schulz_ref(X0.clone(), 5).float()
    ref32 = newton_schulz_ref(X0.float(), 5)
    _status_ok()
    err_ours = ((ours - ref32).norm() / ref32.norm()).item()
    err_ref = ((ref16 - ref32).norm() / ref32.norm()).item()
    assert err_ours < max(2.0 * err_ref, 0.03), (err_ours, err_ref)
    # orthogonality of the result: singular values pushed towards 1
    sv = torch.linalg.svdvals(ours)
    assert sv.max().item() < 1.35 and sv.median().item() > 0.5
    # full pre -> NS -> post against the oracle
    Mr, Sr = M0.clone(), torch.zeros((n, r, 1) if r >= c else (n, 1, c), device="cuda")
    Uref = muon_update_ref(G.clone(), Mr, Sr, 0.9, 0.95, 5).float()
    Mo, So = M0.clone(), torch.zeros_like(Sr)
    X = torch.empty(n, r, c, dtype=torch.bfloat16, device="cuda")
    U = torch.zeros(n, r, c, dtype=torch.bfloat16, device="cuda")
    ln = r if r >= c else c
    sc = torch.empty(3, n, ln, device="cuda")
    sumsq = torch.empty(n, device="cuda")
    cv, ci, cf = _lib.c_void_p, _lib.c_int, _lib.c_float
    _lib.check_rc(_lib.fn("sr_muon_pre", [cv] * 4 + [ci, ci, ci, cf, cf, ci, cv])(
        G.data_ptr(), Mo.data_ptr(), X.data_ptr(), sumsq.data_ptr(), n, r, c, 0.9, 1.0, 1, _lib.stream_ptr()), "pre")
    Xo = newton_schulz_cuda(X, 5, ws)
    from slowrun_b200.optim.muon_adamw import _bf16
    _lib.check_rc(_lib.fn("sr_muon_post", [cv] * 5 + [ci, ci, ci, cf, cv])(
        Xo.data_ptr(), sc[0].data_ptr(), So.data_ptr(), sc[1].data_ptr(), U.data_ptr(), n, r, c, _bf16(0.95), _lib.stream_ptr()), "post")
    _status_ok()
    assert torch.allclose(Mo, Mr, rtol=1e-5, atol=1e-7)
    assert ((U.float() - Uref).norm() / Uref.norm()).item() < 0.1
    assert torch.allclose(So.view(-1), Sr.view(-1), rtol=0.2, atol=1e-6)


def test_muon_apply_and_adamw_kernels():
    from slowrun_b200.optim.muon_adamw import muon_apply_ref, adamw_ref, _bf16
    from slowrun_b200.ops import _lib
    cv, cl, ci, cf = _lib.c_void_p, _lib.ctypes.c_long, _lib.c_int, _lib.c_float
    torch.manual_seed(0)
    P = torch.randn(4, 64, 96, device="cuda") * 0.05
    U = (torch.randn(4, 64, 96, device="cuda") * 0.1).bfloat16()
    Pr = P.clone()
    muon_apply_ref(Pr, U, 0.02, 1.3)
    sh = torch.empty_like(U)
    lr_b = _bf16(0.02)
    _lib.check_rc(_lib.fn("sr_muon_apply", [cv] * 3 + [cl, cf, cf, cv])(P.data_ptr(), U.data_ptr(), sh.data_ptr(), P.numel(), lr_b, _bf16(lr_b * _bf16(1.3)), _lib.stream_ptr()), "apply")
    _status_ok()
    assert torch.allclose(P, Pr, rtol=1e-6, atol=1e-7)
    assert torch.equal(sh, P.bfloat16())
    for dt in (torch.float32, torch.bfloat16):
        p = (torch.randn(1000, 33, device="cuda")).to(dt)
        g = torch.randn(1000, 33, device="cuda") * 0.1
        m = (torch.randn(1000, 33, device="cuda") * 0.01).to(dt)
        v = (torch.rand(1000, 33, device="cuda") * 0.01).to(dt)
        pr, mr, vr = p.clone(), m.clone(), v.clone()
        adamw_ref(pr, g * 0.5, mr, vr, 3, 0.01, 0.8, 0.95, 1e-10, 1.3)
        _lib.check_rc(_lib.fn("sr_adamw", [cv] * 5 + [cl, ci] + [cf] * 8 + [cv])(
            p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), 0, p.numel(), int(dt == torch.bfloat16), 0.01, 1.3, 0.8, 0.95,
            1e-10, 1 - 0.8 ** 3, 1 - 0.95 ** 3, 0.5, _lib.stream_ptr()), "adamw")
        _status_ok()
        tol = 1e-5 if dt == torch.float32 else 2e-2
        assert torch.allclose(p.float(), pr.float(), rtol=tol, atol=tol)
        assert torch.allclose(m.float(), mr.float(), rtol=tol, atol=tol * 0.1)


# ------------------------------------------------------------------ whole model
@pytest.mark.parametrize("track", ["limited", "tiny"])
def test_model_cuda_path_tracks_cpu_oracle(track):
    from slowrun_b200.config import track_defaults
    from slowrun_b200.models.gpt import build_model
    from slowrun_b200.ops import _lib
    cfg = track_defaults(track)
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 4, 256, 2, 2, 256
    m.dropout, m.stoch_depth = 0.0, 0.0
    cpu = build_model(m, "cpu", seed=0)
    gpu = build_model(m, "cuda", seed=0)
    from slowrun_b200.train.checkpoint import load_named_params, named_param_snapshot
    snap = named_param_snapshot(cpu)
    torch.manual_seed(1)
    for k in snap:   # move gates / mixes / lambdas off their neutral init
        if any(s in k for s in ("gate", "mix", "lambdas", "skip", "xsa")):
            snap[k] = snap[k] + 0.05 * torch.randn_like(snap[k])
    load_named_params(cpu, snap)
    load_named_params(gpu, snap)
    cpu.norm_eps = gpu.norm_eps
    idx = torch.randint(0, 50257, (2, 256))
    tgt = torch.randint(0, 50257, (2, 256))
    kw = {}
    if track == "tiny":
        kw = dict(num_iterations=2, mtp_weights=torch.tensor([1.0, 0.5, 0.25]))
    cpu.train(); gpu.train()
    out_c = cpu(idx, tgt, **kw)
    gkw = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in kw.items()}
    out_g = gpu(idx.cuda(), tgt.cuda(), **gkw)
    lc = out_c[0] if isinstance(out_c, tuple) else out_c
    lg = out_g[0] if isinstance(out_g, tuple) else out_g
    lc.backward(); lg.backward()
    torch.cuda.synchronize(); _lib.check_status()
    assert abs(lc.item() - lg.item()) < 0.05, (lc.item(), lg.item())
    # gradient direction agreement on the big matrices (bf16 activations vs fp32 oracle)
    for (n, pc), (_, pg) in zip(cpu.named_parameters(), gpu.named_parameters()):
        gc = cpu.arena.head_grad if n == "lm_head.weight" else pc.grad
        gg = gpu.arena.head_grad if n == "lm_head.weight" else pg.grad
        if gc is None or gc.abs().max() == 0 or pc.dim() < 2 or pc.numel() < 4096:
            continue
        cos = torch.nn.functional.cosine_similarity(gc.flatten().float(), gg.flatten().float().cpu(), dim=0).item()
        assert cos > 0.97, (n, cos)


def test_graft_smoke():
    import __graft_entry__ as g
    g.smoke()


@pytest.mark.parametrize("track", ["limited", "tiny"])
def test_fused_block_node_matches_op_by_op_path(track):
    """Same CUDA model, block run as one autograd node vs. op by op: loss and every gradient must agree. The tiny
    configuration adds the key offset (layer 3 is a long-window layer) and exclusive self-attention on every layer."""
    from slowrun_b200.config import track_defaults
    from slowrun_b200.models.gpt import build_model
    from slowrun_b200.ops import _lib
    cfg = track_defaults(track)
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 4, 256, 2, 2, 256
    m.dropout, m.stoch_depth = 0.0, 0.0
    model = build_model(m, "cuda", seed=0)
    torch.manual_seed(1)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if any(s in n for s in ("gate", "mix", "lambdas", "skip", "xsa")):
                p.add_(0.05 * torch.randn_like(p))
            if track == "tiny" and "c_proj" in n:       # zero-initialised in this track: nothing would flow back
                p.add_(0.02 * torch.randn_like(p))
        if track == "tiny":
            model.xsa_alphas.add_(0.5)
    model.arena.refresh_shadows()
    if track == "limited":
        model.set_dupe_layers(2, 3, 1)
    idx = torch.randint(0, 50257, (2, 256), device="cuda")
    tgt = torch.randint(0, 50257, (2, 256), device="cuda")
    kw = dict(num_iterations=2, mtp_weights=torch.tensor([1.0, 0.5, 0.25], device="cuda")) if track == "tiny" else {}
    res = {}
    for fused in (True, False):
        model.use_fused_blocks = fused
        model.zero_grad_arena()
        out = model(idx, tgt, **kw)
        loss = out[0] if isinstance(out, tuple) else out
        loss.backward()
        torch.cuda.synchronize(); _lib.check_status()
        res[fused] = (loss.item(), {n: (model.arena.head_grad if n == "lm_head.weight" else p.grad).clone()
                                    for n, p in model.named_parameters()})
    assert abs(res[True][0] - res[False][0]) < 2e-2, (res[True][0], res[False][0])
    for n in res[True][1]:
        a, b = res[True][1][n].float(), res[False][1][n].float()
        if b.abs().max() == 0:
            assert a.abs().max() == 0, n
            continue
        cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
        if a.numel() < 4096:      # tiny tensors (mixes, gates, scalars) carry round-off-sized gradients here
            assert cos > 0.9, (n, cos)
            continue
        assert cos > 0.99, (n, cos)
        assert abs(a.norm().item() / b.norm().item() - 1) < 0.1, (n, a.norm().item(), b.norm().item())


def test_fused_block_with_dropout_and_stochastic_depth_runs():
    from slowrun_b200.config import track_defaults
    from slowrun_b200.models.gpt import build_model
    from slowrun_b200.ops import _lib
    cfg = track_defaults("limited")
    m = cfg.model
    m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 4, 256, 2, 2, 128
    m.stoch_depth = 0.5
    model = build_model(m, "cuda", seed=0)
    idx = torch.randint(0, 50257, (2, 128), device="cuda")
    for _ in range(3):
        loss, _ = model(idx, idx)
        loss.backward()
    torch.cuda.synchronize(); _lib.check_status()
    assert torch.isfinite(loss)
    for n, p in model.named_parameters():
        assert torch.isfinite(p.grad.float()).all(), n


@pytest.mark.parametrize("B,T,H,window", [(1, 128, 1, -1), (2, 384, 3, -1), (1, 2048, 2, 1024), (2, 2047, 2, -1),
                                           (1, 1000, 2, 256), (1, 640, 1, 100)])
@pytest.mark.parametrize("bkv", [64, 128])
def test_native_flash_attention_forward(B, T, H, window, bkv):
    from slowrun_b200.ops.flash_attention import native_available, native_fwd
    from slowrun_b200.ops.functional import attention_ref
    if not native_available():
        pytest.skip("native attention not built")
    q, k, v = _bf(B, T, H, 128, seed=21), _bf(B, T, H, 128, seed=22), _bf(B, T, H, 128, seed=23)
    out, lse, sc, w = native_fwd(q, k, v, window, None, bkv=bkv)
    _status_ok()
    ref = attention_ref(q.float(), k.float(), v.float(), window, None)
    _close(out, ref, 3e-2, 3e-2)
    # log-sum-exp of the scaled scores
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * (128 ** -0.5)
    i = torch.arange(T, device="cuda").unsqueeze(1)
    j = torch.arange(T, device="cuda").unsqueeze(0)
    mask = (j <= i) & ((i - j) <= (window if window >= 0 else T))
    s = s.masked_fill(~mask, float("-inf"))
    assert torch.allclose(lse, torch.logsumexp(s, dim=-1), rtol=1e-3, atol=1e-2)


def test_native_flash_attention_on_strided_qkv_view():
    from slowrun_b200.ops.flash_attention import native_available, native_fwd
    from slowrun_b200.ops.functional import attention_ref
    if not native_available():
        pytest.skip("native attention not built")
    B, T, H = 2, 256, 2
    qkv = _bf(B, T, 3, H, 128, seed=24)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    out, *_ = native_fwd(q, k, v, 64, 0.1)
    _status_ok()
    _close(out, attention_ref(q.float(), k.float(), v.float(), 64, 0.1), 3e-2, 3e-2)


@pytest.mark.parametrize("B,T,H,window", [(1, 128, 1, -1), (2, 384, 2, -1), (1, 1024, 2, 256), (1, 2047, 1, -1), (1, 700, 2, 100)])
def test_native_flash_attention_backward(B, T, H, window):
    from slowrun_b200.ops.flash_attention import native_available, native_fwd, native_bwd, _has
    from slowrun_b200.ops.functional import attention_ref
    if not (native_available() and _has("sr_flash_attn_bwd")):
        pytest.skip("native attention backward not built")
    q, k, v = _bf(B, T, H, 128, seed=31), _bf(B, T, H, 128, seed=32), _bf(B, T, H, 128, seed=33)
    dy = _bf(B, T, H, 128, seed=34)
    out, lse, sc, w = native_fwd(q, k, v, window, None)
    dq, dk, dv = native_bwd(dy, q, k, v, out, lse, sc, w)
    _status_ok()
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ref = attention_ref(qf, kf, vf, window, None)
    ref.backward(dy.float())
    _close(dq, qf.grad, 4e-2, 4e-2)
    _close(dk, kf.grad, 4e-2, 4e-2)
    _close(dv, vf.grad, 4e-2, 4e-2)


def test_cuda_graph_micro_step_matches_eager(tmp_path):
    """Trainer with captured micro-steps must reproduce the eager run (dropout and stochastic depth off)."""
    from slowrun_b200.config import track_defaults
    from slowrun_b200.data.synthetic import write_synthetic_corpus
    from slowrun_b200.parallel.comm import DistInfo
    from slowrun_b200.train.trainer import Trainer
    tr_path, va_path = write_synthetic_corpus(str(tmp_path), train_tokens=300_000, val_tokens=20_000)
    finals = {}
    for graphs in (False, True):
        cfg = track_defaults("limited")
        m = cfg.model
        m.n_layer, m.n_embd, m.n_head, m.n_kv_head, m.sequence_len = 4, 256, 2, 2, 256
        m.dropout, m.stoch_depth = 0.0, 0.0
        cfg.device_batch_size, cfg.total_batch_size = 2, 2 * 256 * 4
        cfg.input_bin, cfg.input_val_bin, cfg.cuda_graphs = tr_path, va_path, graphs
        t = Trainer(cfg, DistInfo(False, 0, 0, 1, torch.device("cuda", 0)), quiet=True)
        losses = [t.train_step()["loss"] for _ in range(4)]
        assert t.use_graphs == graphs and (len(t._graphs) == 1) == graphs
        finals[graphs] = (losses, {n: p.detach().float().clone() for n, p in t.model.named_parameters()})
    for a, b in zip(finals[True][0], finals[False][0]):
        assert abs(a - b) < 5e-2, (finals[True][0], finals[False][0])
    num = sum((finals[True][1][n] - finals[False][1][n]).pow(2).sum() for n in finals[True][1])
    den = sum(finals[False][1][n].pow(2).sum() for n in finals[False][1])
    assert (num / den).sqrt().item() < 2e-2


@pytest.mark.parametrize("H,J", [(20, 128 * 2560), (14, 128 * 1792), (8, 4096 + 66), (2, 1000)])
def test_iha_mixing_kernels(H, J):
    from slowrun_b200.ops.block import iha_mix_weights, iha_mix_backward
    P = 3
    mixes = (torch.eye(H, device="cuda").expand(P, H, H) + 0.1 * torch.randn(P, H, H, device="cuda")).contiguous()
    w = _bf(P * H, J, scale=0.05, seed=41)
    out = iha_mix_weights(mixes, w, H)
    ref = torch.bmm(mixes.bfloat16().float(), w.view(P, H, J).float())
    _status_ok()
    _close(out.view(P, H, J), ref)
    dwp = _bf(P * H, J, scale=0.01, seed=42)
    gw = torch.randn(P * H, J, device="cuda")
    gw_ref = gw.view(P, H, J) + torch.bmm(mixes.bfloat16().float().transpose(1, 2), dwp.view(P, H, J).float())
    dmix = iha_mix_backward(mixes, w, dwp, gw, H)
    _status_ok()
    dmix_ref = torch.bmm(dwp.view(P, H, J).float(), w.view(P, H, J).float().transpose(1, 2))
    assert torch.allclose(gw.view(P, H, J), gw_ref, rtol=1e-3, atol=1e-3)
    assert torch.allclose(dmix, dmix_ref, rtol=2e-3, atol=2e-3 * dmix_ref.abs().max().item())


@pytest.mark.parametrize("nc,scale", [(12, 1.0), (32, 2.0)])
def test_per_head_gate_kernels(nc, scale):
    """gate = scale * sigmoid(a[:, :nc] @ bf16(W)^T) and its backward (weight gradient accumulated, input gradient added)."""
    from slowrun_b200.ops.block import _gate_bwd, _gate_fwd
    M, C, H = 1000, 256, 20
    a = _bf(M, C, seed=51)
    w = torch.nn.Parameter(torch.randn(H, nc, device="cuda") * 0.3)
    gate = _gate_fwd(a, w.data, H, nc, scale)
    af = a.float().requires_grad_(True)
    wf = w.detach().bfloat16().float().requires_grad_(True)
    z = (af[:, :nc] @ wf.t()).bfloat16().float()
    ref = scale * torch.sigmoid(z)
    _status_ok()
    assert torch.allclose(gate, ref, rtol=1e-3, atol=1e-3)
    dg = torch.randn(M, H, device="cuda")
    zz = af[:, :nc] @ wf.t()
    (scale * torch.sigmoid(zz) * dg).sum().backward()
    w.grad = torch.full_like(w, 0.5)
    da = _bf(M, C, seed=52)
    da0 = da.clone()
    _gate_bwd(dg, gate, a, w, da, H, nc, scale)
    _status_ok()
    assert torch.allclose(w.grad - 0.5, wf.grad, rtol=2e-2, atol=2e-2 * wf.grad.abs().max().item())
    assert torch.equal(da[:, nc:], da0[:, nc:])
    _close(da[:, :nc].float() - da0[:, :nc].float(), af.grad[:, :nc], 4e-2, 4e-2)


def test_attention_backward_with_gate_delta_and_fp32_dq():
    """The fused-block form of the attention backward: delta comes out of the head-gate backward, dQ stays in fp32."""
    from slowrun_b200.ops import _lib
    from slowrun_b200.ops.block import P, I, L, _call, _sp
    from slowrun_b200.ops.flash_attention import _has, native_available, native_bwd, native_fwd
    if not (native_available() and _has("sr_flash_attn_bwd_ex")):
        pytest.skip("native attention backward not built")
    B, T, H, D = 2, 512, 3, 128
    q, k, v = _bf(B, T, H, D, seed=61), _bf(B, T, H, D, seed=62), _bf(B, T, H, D, seed=63)
    y, lse, sc, w = native_fwd(q, k, v, 200, None)
    gate = torch.rand(B * T, H, device="cuda")
    dy2 = _bf(B, T, H, D, seed=64)
    dy = torch.empty_like(y)
    dgate = torch.empty(B * T, H, device="cuda")
    delta = torch.empty(B, H, T, device="cuda")
    _call("sr_head_gate_bwd_delta", [P] * 6 + [L, I, I, L, L, L, P], dy2.data_ptr(), y.data_ptr(), gate.data_ptr(), dy.data_ptr(),
          dgate.data_ptr(), delta.data_ptr(), B * T, H, T, H * D, H * D, H * D, _sp())
    _status_ok()
    delta_ref = (dy.float() * y.float()).sum(-1).permute(0, 2, 1)
    assert torch.allclose(delta, delta_ref, rtol=2e-2, atol=2e-2 * delta_ref.abs().max().item())
    dq32, dk, dv = native_bwd(dy, q, k, v, y, lse, sc, w, delta=delta, dq_fp32=True)
    dq, dk2, dv2 = native_bwd(dy, q, k, v, y, lse, sc, w)
    _status_ok()
    assert dq32.dtype == torch.float32
    _close(dq32, dq, 2e-2, 2e-2)
    _close(dk, dk2, 2e-2, 2e-2)
    _close(dv, dv2, 2e-2, 2e-2)
