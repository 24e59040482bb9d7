"""Kernel micro-benchmarks (CUDA-event timed, warm-up, L2 flushed between iterations) and the small fixed workloads
that the ncu captures under profiles/ are taken on.

    python -m slowrun_b200.bench.kernels gemm --m 8192 --n 7680 --k 2560 [--a-mn] [--b-mn] [--acc] [--iters 20]
    python -m slowrun_b200.bench.kernels attn --b 4 --t 2048 --h 20 --window 1024 [--bwd]
    python -m slowrun_b200.bench.kernels ce --m 8192 --v 50304
    python -m slowrun_b200.bench.kernels ns --n 4 --r 2560 --c 2560
    python -m slowrun_b200.bench.kernels lmhead_ce --m 16384 --d 2560 --v 50304 [--fp8]
    python -m slowrun_b200.bench.kernels rowwise --m 8192 --d 2560        (memory-bound glue kernels, one line each)
    python -m slowrun_b200.bench.kernels optim --n 8 --r 2560 --c 2560    (Muon prologue / apply, AdamW)
Prints one JSON line per run with the achieved rate and its fraction of the measured peaks in MEASURED_PEAKS.json
(fallback 6.65 TB/s, 1590 TFLOP/s when the file is absent).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    try:
        d = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, 1590.0, "fallback"


def timed(fn, iters, flush=True):
    scratch = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if scratch is not None:
            scratch.zero_()          # 160 MB write: evicts the 126 MB L2
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def _reference_head(a):
    """The reference's formulation of the same op (tiny/cuda_kernels.py:338-414: three torch._scaled_mm products, its
    NVRTC loss kernel and its Triton transposes), loaded unmodified from the reference tree. Its loss kernel is
    compiled for sm_90 only, so the one call that compiles it is redirected to this GPU's architecture from here, the
    file itself is untouched. Returns (callable, None) or (None, reason)."""
    import importlib.util
    ref = os.environ.get("SLOWRUN_REFERENCE_DIR") or os.path.join(ROOT, "baseline", "_ref")
    path = os.path.join(ref, "tiny", "cuda_kernels.py")
    if not os.path.isfile(path):
        return None, f"{path} not present"
    if a.v != 50304:
        return None, "the reference loss kernel is compiled for a vocabulary of exactly 50304"
    orig = torch.cuda._compile_kernel
    cc = "".join(str(x) for x in torch.cuda.get_device_capability())

    def compile_for_this_gpu(*args, **kw):
        kw["compute_capability"] = cc
        return orig(*args, **kw)

    try:
        torch.cuda._compile_kernel = compile_for_this_gpu
        spec = importlib.util.spec_from_file_location("ref_tiny_cuda_kernels", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    except Exception as e:  # noqa: BLE001
        return None, f"{type(e).__name__}: {str(e).splitlines()[0] if str(e) else ''}"[:200]
    finally:
        torch.cuda._compile_kernel = orig
    return mod.FusedSoftcappedCrossEntropy, None


def lmhead_ce_bench(a, hbm, tf):
    """lm-head + soft-capped CE, forward and backward (dx and dW), at [m tokens, d] x [v, d]: the fused kernels
    against this library's own GEMM -> logits -> loss-kernel path and against the reference's formulation."""
    from slowrun_b200.ops import functional as ops
    M, d, V = a.m, a.d, a.v
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(M, d, device="cuda", generator=g).bfloat16()
    w = (torch.randn(V, d, device="cuda", generator=g) * 0.02).bfloat16()
    tgt = torch.randint(0, V - 47, (M,), device="cuda", generator=g)
    acc = torch.zeros(V, d, device="cuda", dtype=torch.float32)
    vocab = V - 47 if V == 50304 else V
    res = {"shape": [M, d, V], "fp8": bool(a.fp8)}

    def ours(fused, fp8):
        def step():
            ops.set_fused_head(fused)
            xa = x.detach().requires_grad_(not a.fwd_only)
            loss = ops.lm_head_loss(xa, w, tgt, 15.0, vocab, grad_acc=acc, fp8=fp8)
            if not a.fwd_only:
                loss.backward()
            ops.set_fused_head(True)
        return step

    ms_fused = timed(ours(True, a.fp8), a.iters, not a.no_flush)
    res["ms_fused"] = ms_fused
    if a.fwd_only:
        fl = 2.0 * M * d * V
        res.update(tflops=fl / ms_fused / 1e9, frac_of_peak=fl / ms_fused / 1e9 / tf)
        return res
    ms_unfused = timed(ours(False, False), a.iters, not a.no_flush)
    fl = 3 * 2.0 * M * d * V
    # roofline: three products at the measured bf16 rate (the fp8 forward could run at twice that), or the bytes that
    # must move (E' written once and read twice, operands and gradients once) at the measured copy rate
    byts = 3.0 * M * V * 2 + 2.0 * M * d * 2 * 2 + V * d * (2 + 8)
    t_roof = max(fl / (tf * 1e9), byts / (hbm * 1e6))
    res.update(ms_unfused=ms_unfused, speedup_vs_unfused=ms_unfused / ms_fused, tflops=fl / ms_fused / 1e9,
               roofline_ms=t_roof, frac_of_roofline=t_roof / ms_fused)
    ref_fn, why = _reference_head(a)
    if ref_fn is None:
        res["reference"] = {"unavailable": why}
        return res
    try:
        wt = w.t().contiguous()                 # the tiny track stores the head as [d, V]
        wts = torch.tensor([1.0], device="cuda")

        def ref_step():
            xa = x.detach().requires_grad_(True)
            wa = wt.detach().requires_grad_(True)
            losses = ref_fn.apply(xa, tgt, wts, wa, ops.FP8_X_SCALE, ops.FP8_W_SCALE, 0.75 / 448, 1.0 / M, 15.0)
            losses.mean().backward()

        ms_ref = timed(ref_step, a.iters, not a.no_flush)
        res["reference"] = {"ms": ms_ref, "what": "tiny/cuda_kernels.py FusedSoftcappedCrossEntropy fwd+bwd (fp8 _scaled_mm x3)"}
        res["speedup_vs_reference"] = ms_ref / ms_fused
    except Exception as e:  # noqa: BLE001
        res["reference"] = {"unavailable": f"{type(e).__name__}: {str(e).splitlines()[0] if str(e) else ''}"[:200]}
    return res


def rowwise_bench(a, hbm):
    """The memory-bound kernels between the GEMMs on [m, d] activations; bytes = tensors each op must read and write once."""
    from slowrun_b200.ops import functional as ops
    M, d, dev = a.m, a.d, "cuda"
    bf = lambda *s: torch.randn(*s, device=dev).bfloat16()
    x, y, x0 = bf(M, d), bf(M, d), bf(M, d)
    gf = bf(M, 2 * 4 * d // 2)                       # [gate | fc] for a SwiGLU of hidden size 2d (any even split works)
    res = []

    def add(name, fn, nbytes, bwd_of=None):
        if bwd_of is not None:
            outp = bwd_of()
            g = torch.randn_like(outp)
            fn = lambda: torch.autograd.grad(outp, inputs, g, retain_graph=True)
        ms = timed(fn, a.iters, not a.no_flush)
        res.append({"kernel": name, "ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1),
                    "frac_of_copy_peak": round(nbytes / ms / 1e6 / hbm, 3)})

    e = 2.0 * M * d                                   # bytes of one bf16 [m, d] tensor
    add("rms_norm_fwd", lambda: ops.rms_norm(x), 2 * e)
    add("swiglu_fwd", lambda: ops.swiglu(gf), 2.0 * gf.numel() + gf.numel())
    inputs = [gf.clone().requires_grad_(True)]
    add("swiglu_bwd", None, 2.0 * gf.numel() * 2 + gf.numel(), bwd_of=lambda: ops.swiglu(inputs[0]))
    add("dropout_add_fwd(p=0.1)", lambda: ops.dropout_add(x, y, 0.1, True), 3 * e)
    lam = torch.ones(4, device=dev)
    add("lambda_mix_fwd", lambda: ops.lambda_mix(x, x0, None, lam, lam, lam, 0, 0), 3 * e)
    H = max(1, d // 128)
    q = bf(1, M, H, 128)
    cos, sin = torch.randn(1, M, 1, 64, device=dev).bfloat16(), torch.randn(1, M, 1, 64, device=dev).bfloat16()
    add("rope_qknorm_fwd", lambda: ops.rope_qknorm(q, cos, sin), 2.0 * q.numel() * 2)
    # the fused block kernels, called as the block node calls them (T = 2048 tokens per sequence)
    from slowrun_b200.ops import _lib
    P, I, L, F32, ULL = _lib.c_void_p, _lib.c_int, ctypes.c_long, _lib.c_float, ctypes.c_ulonglong
    sp = _lib.stream_ptr
    T = 2048 if M % 2048 == 0 else M
    C = H * 128
    eps = 1e-6
    scal = torch.tensor([1.1, 0.2, 0.7], device=dev)
    xa, xb, sk = bf(M, d), bf(M, d), bf(M, d)
    o1, o2 = torch.empty_like(xa), torch.empty_like(xa)
    f = _lib.fn("sr_mix_norm_fwd", [P] * 8 + [L, I, F32, P])
    add("mix_norm_fwd (lambda mix + skip + RMSNorm)",
        lambda: f(xa.data_ptr(), xb.data_ptr(), sk.data_ptr(), o1.data_ptr(), o2.data_ptr(), scal.data_ptr(), scal.data_ptr() + 4,
                  scal.data_ptr() + 8, M, d, eps, sp()), 5 * e)
    f2 = _lib.fn("sr_add_norm_fwd", [P] * 4 + [L, I, F32, F32, ULL, P, P])
    st = ops.dropout_state(dev)
    add("add_norm_fwd (residual + dropout + RMSNorm)",
        lambda: f2(xa.data_ptr(), xb.data_ptr(), o1.data_ptr(), o2.data_ptr(), M, d, eps, 0.1, 12345, st.data_ptr(), sp()), 4 * e)
    qkv, ve = bf(M, 3 * C), bf(M, C)
    gate = torch.rand(M, H, device=dev) * 2
    ang = torch.rand(T, 64, device=dev) * 6.28
    c2, s2 = ang.cos().bfloat16(), ang.sin().bfloat16()
    qo, ko, vo = (torch.empty(M // T, T, H, 128, dtype=torch.bfloat16, device=dev) for _ in range(3))
    f3 = _lib.fn("sr_qkv_prep_fwd", [P] * 8 + [L, I, I, F32, I, P])
    add("qkv_prep_fwd (split + value residual + RoPE + QK-norm + key offset)",
        lambda: f3(qkv.data_ptr(), ve.data_ptr(), gate.data_ptr(), c2.data_ptr(), s2.data_ptr(), qo.data_ptr(), ko.data_ptr(),
                   vo.data_ptr(), M, H, T, eps, 1, sp()), 2.0 * M * C * (3 + 1 + 3))
    alpha = torch.linspace(-0.5, 0.5, H, device=dev)
    g01 = torch.rand(M, H, device=dev)
    f4 = _lib.fn("sr_attn_post_fwd", [P] * 5 + [L, I, F32, P])
    add("attn_post_fwd (head gate + XSA projection)",
        lambda: f4(qo.data_ptr(), vo.data_ptr(), g01.data_ptr(), alpha.data_ptr(), ko.data_ptr(), M, H, 1e-4, sp()), 2.0 * M * C * 3)
    return {"shape": [M, d], "kernels": res}


def optim_bench(a, hbm):
    """Single-GPU optimizer kernels on a stack of n matrices [r, c]: bytes = every state tensor read and written once."""
    from slowrun_b200.ops import _lib
    P, I, F, L = _lib.c_void_p, _lib.c_int, _lib.c_float, ctypes.c_long
    n, r, c, dev = a.n if a.n <= 64 else 8, a.r, a.c, "cuda"
    N = n * r * c
    G = torch.randn(n, r, c, device=dev) * 0.02
    Mom, X, ss = torch.zeros_like(G), torch.empty(n, r, c, device=dev, dtype=torch.bfloat16), torch.zeros(n, device=dev)
    Pm, U, W16 = torch.randn(n, r, c, device=dev), torch.randn(n, r, c, device=dev).bfloat16(), torch.empty(n, r, c, device=dev, dtype=torch.bfloat16)
    res = []

    def add(name, fn, nbytes):
        ms = timed(fn, a.iters, not a.no_flush)
        res.append({"kernel": name, "ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1),
                    "frac_of_copy_peak": round(nbytes / ms / 1e6 / hbm, 3)})

    pre = _lib.fn("sr_muon_pre", [P] * 4 + [I, I, I, F, F, I, P])
    add("muon_pre (grad -> momentum, Nesterov, row norm, bf16 X)",
        lambda: pre(G.data_ptr(), Mom.data_ptr(), X.data_ptr(), ss.data_ptr(), n, r, c, 0.95, 1.0, 1, _lib.stream_ptr()),
        N * (4 + 4 + 4 + 2.0))                        # G read, momentum read+write, X write (second pass served by L2 or re-read)
    app = _lib.fn("sr_muon_apply", [P] * 3 + [L, F, F, P])
    add("muon_apply (cautious weight decay + bf16 shadow)",
        lambda: app(Pm.data_ptr(), U.data_ptr(), W16.data_ptr(), N, 0.02, 0.002, _lib.stream_ptr()), N * (4 + 4 + 2 + 2.0))
    m_, v_ = torch.zeros(N, device=dev), torch.zeros(N, device=dev)
    adam = _lib.fn("sr_adamw", [P] * 5 + [L, I] + [F] * 8 + [P])
    add("adamw (fp32 state + bf16 shadow)",
        lambda: adam(Pm.data_ptr(), G.data_ptr(), m_.data_ptr(), v_.data_ptr(), W16.data_ptr(), N, 0, 1e-3, 0.1, 0.8, 0.95, 1e-10,
                     0.2, 0.05, 1.0, _lib.stream_ptr()), N * (4 * 2 + 4 + 4 * 2 + 4 * 2 + 2.0))
    return {"shape": [n, r, c], "kernels": res}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attn", "ce", "ns", "lmhead_ce", "rowwise", "optim"])
    ap.add_argument("--d", type=int, default=2560)
    ap.add_argument("--fp8", action="store_true", help="lmhead_ce: e4m3 forward product (per-tensor scales)")
    ap.add_argument("--fwd-only", action="store_true", help="lmhead_ce: time only the forward (the small ncu workload)")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=7680)
    ap.add_argument("--k", type=int, default=2560)
    ap.add_argument("--a-mn", action="store_true")
    ap.add_argument("--b-mn", action="store_true")
    ap.add_argument("--acc", action="store_true", help="fp32 accumulate-into output (weight-gradient form)")
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--b", type=int, default=4)
    ap.add_argument("--t", type=int, default=2048)
    ap.add_argument("--h", type=int, default=20)
    ap.add_argument("--window", type=int, default=-1)
    ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--v", type=int, default=50304)
    ap.add_argument("--r", type=int, default=2560)
    ap.add_argument("--c", type=int, default=2560)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--no-pair", action="store_true", help="GEMMs on the single-CTA kernel only")
    a = ap.parse_args()
    sys.path.insert(0, ROOT)
    from slowrun_b200.ops import _lib
    from slowrun_b200.ops.gemm import gemm, set_pair_mode
    if a.no_pair:
        set_pair_mode(False)
    hbm, tf, src = peaks()
    out = {"what": a.what, "peaks": src}
    if a.what == "gemm":
        A = torch.randn((a.k, a.m) if a.a_mn else (a.m, a.k), device="cuda").bfloat16() * 0.1
        B = torch.randn((a.k, a.n) if a.b_mn else (a.n, a.k), device="cuda").bfloat16() * 0.1
        C = torch.zeros(a.m, a.n, device="cuda", dtype=torch.float32 if a.acc else torch.bfloat16)
        if a.acc:
            fn = lambda: gemm(A, B, out=C, cin=C, a_mn=a.a_mn, b_mn=a.b_mn, beta=1.0, bn=a.bn)
        else:
            fn = lambda: gemm(A, B, out=C, a_mn=a.a_mn, b_mn=a.b_mn, bn=a.bn)
        ms = timed(fn, a.iters, not a.no_flush)
        fl = 2.0 * a.m * a.n * a.k
        out.update(shape=[a.m, a.n, a.k], ms=ms, tflops=fl / ms / 1e9, frac_of_peak=fl / ms / 1e9 / tf)
    elif a.what == "attn":
        from slowrun_b200.ops.flash_attention import native_bwd, native_fwd
        q, k, v = (torch.randn(a.b, a.t, a.h, 128, device="cuda", dtype=torch.bfloat16) for _ in range(3))
        keys = sum(min(i, a.window if a.window >= 0 else i) + 1 for i in range(a.t))
        fl = 4.0 * a.b * a.h * keys * 128
        o, lse, sc, w = native_fwd(q, k, v, a.window, None)
        if a.bwd:
            dy = torch.randn_like(o)
            ms = timed(lambda: native_bwd(dy, q, k, v, o, lse, sc, w), a.iters, not a.no_flush)
            fl *= 2.5
        else:
            ms = timed(lambda: native_fwd(q, k, v, a.window, None), a.iters, not a.no_flush)
        out.update(shape=[a.b, a.t, a.h, 128], window=a.window, bwd=a.bwd, ms=ms, tflops=fl / ms / 1e9, frac_of_peak=fl / ms / 1e9 / tf)
    elif a.what == "ce":
        from slowrun_b200.ops import functional as ops
        logits = torch.randn(a.m, a.v, device="cuda").bfloat16()
        tgt = torch.randint(0, a.v - 64, (a.m,), device="cuda")
        loss = torch.empty(a.m, device="cuda")
        scale = torch.full((), 1.0 / a.m, device="cuda")
        fn = lambda: ops._call("sr_softcap_ce", ops._CE_ARGS, logits.data_ptr(), tgt.data_ptr(), loss.data_ptr(), 0, 1,
                               scale.data_ptr(), a.m, a.v, a.v - 47, a.v, 10.0, 1, _lib.stream_ptr())
        ms = timed(fn, a.iters, not a.no_flush)
        byts = a.m * a.v * 2 * 2.0      # one read from HBM, one write (second read is served by L2)
        out.update(shape=[a.m, a.v], ms=ms, gbs=byts / ms / 1e6, frac_of_peak=byts / ms / 1e6 / hbm)
    elif a.what == "lmhead_ce":
        out.update(lmhead_ce_bench(a, hbm, tf))
    elif a.what == "rowwise":
        out.update(rowwise_bench(a, hbm))
    elif a.what == "optim":
        out.update(optim_bench(a, hbm))
    else:
        from slowrun_b200.optim.muon_adamw import _NSWorkspace, newton_schulz_cuda, newton_schulz_ref
        X = (torch.randn(a.n, a.r, a.c, device="cuda") / (a.r * a.c) ** 0.5).bfloat16()
        ws = _NSWorkspace(a.n, a.r, a.c, "cuda")
        ms = timed(lambda: newton_schulz_cuda(X.clone(), 5, ws), a.iters, not a.no_flush)
        # the same five iterations as the reference runs them: 15 batched bf16 products through the library
        ms_lib = timed(lambda: newton_schulz_ref(X.clone(), 5), a.iters, not a.no_flush)
        g, o = min(a.r, a.c), max(a.r, a.c)
        fl = 5 * a.n * (4.0 * g * g * o + 2.0 * g ** 3)      # full (non-symmetric) cost, the reference's bmm count
        out.update(shape=[a.n, a.r, a.c], ms=ms, ms_library_bmm=ms_lib, speedup_vs_library=ms_lib / ms,
                   tflops_equiv=fl / ms / 1e9, frac_of_peak=fl / ms / 1e9 / tf)
    torch.cuda.synchronize()
    _lib.check_status()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
