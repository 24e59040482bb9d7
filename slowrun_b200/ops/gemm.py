"""Python face of the tcgen05 bf16 GEMM (`csrc/gemm_tcgen05.cu`) plus its plain-PyTorch reference.

`gemm()` computes ``out[b] = alpha * op(A[b]) @ op(B[b]).T + beta * cin[b]`` with A an (M x K) operand and B an
(N x K) operand. Each operand is given as stored: ``a_mn=False`` means the tensor is [.., M, K] (K contiguous),
``a_mn=True`` means it is [.., K, M] (M contiguous). The reference reaches cuBLAS for the same products through
F.linear / torch.bmm (train.py:286-323, 614-621).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_ARGTYPES = [
    _lib.c_void_p, _lib.c_void_p, _lib.c_void_p, _lib.c_void_p,  # A B C Cin
    _lib.c_int, _lib.c_int, _lib.c_int, _lib.c_int,  # M N K batch
    _lib.c_ll, _lib.c_ll, _lib.c_ll, _lib.c_ll,  # lda ldb ldc ldcin
    _lib.c_ll, _lib.c_ll, _lib.c_ll, _lib.c_ll,  # strides
    _lib.c_int, _lib.c_int, _lib.c_int, _lib.c_int,  # a_mn b_mn c_fp32 cin_fp32
    _lib.c_float, _lib.c_float, _lib.c_void_p, _lib.c_void_p,  # alpha beta alpha_ptr row_scale
    _lib.c_int, _lib.c_int, _lib.c_int,  # sym bn max_ctas
    _lib.c_void_p, _lib.c_void_p,  # status stream
]


def _as3d(t: torch.Tensor):
    if t.dim() == 2:
        return t.unsqueeze(0)
    if t.dim() == 3:
        return t
    raise ValueError(f"expected a 2-D or 3-D tensor, got {tuple(t.shape)}")


def _check_operand(t: torch.Tensor, name: str):
    if t.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be bfloat16, got {t.dtype}")
    if t.stride(-1) != 1:
        raise ValueError(f"{name} must have a contiguous last dimension")


def gemm_reference(a, b, cin=None, *, a_mn=False, b_mn=False, alpha=1.0, beta=0.0, out_dtype=torch.bfloat16,
                   row_scale=None):
    """fp32 PyTorch statement of `gemm` (the numerics oracle; runs on CPU or GPU)."""
    A = _as3d(a).float()
    B = _as3d(b).float()
    if a_mn:
        A = A.transpose(-1, -2)
    if b_mn:
        B = B.transpose(-1, -2)
    out = alpha * torch.matmul(A, B.transpose(-1, -2))
    if row_scale is not None:
        out = out * row_scale.float().reshape(out.shape[0], -1, 1)
    if cin is not None:
        out = out + beta * _as3d(cin).float()
    out = out.to(out_dtype)
    return out if a.dim() == 3 else out[0]


def gemm(a, b, out=None, cin=None, *, a_mn=False, b_mn=False, alpha=1.0, beta=0.0, alpha_t=None, sym=False,
         out_dtype=torch.bfloat16, bn=0, max_ctas=0, row_scale=None):
    """Launch the tcgen05 GEMM on the current stream. See the module docstring for operand conventions.

    `alpha_t` is an optional 0-dim fp32 CUDA tensor multiplied into alpha on the device (no host sync);
    `row_scale` an optional fp32 CUDA tensor [batch, M] (or [M]) that scales the rows of the product."""
    if alpha_t is not None and (alpha_t.dtype != torch.float32 or not alpha_t.is_cuda):
        raise TypeError("alpha_t must be a float32 CUDA tensor")
    if row_scale is not None and (row_scale.dtype != torch.float32 or not row_scale.is_cuda
                                  or not row_scale.is_contiguous()):
        raise TypeError("row_scale must be a contiguous float32 CUDA tensor")
    _check_operand(a, "a")
    _check_operand(b, "b")
    A, B = _as3d(a), _as3d(b)
    batch = A.shape[0]
    if a_mn:
        K, M = A.shape[1], A.shape[2]
    else:
        M, K = A.shape[1], A.shape[2]
    if b_mn:
        Kb, N = B.shape[1], B.shape[2]
    else:
        N, Kb = B.shape[1], B.shape[2]
    if Kb != K or B.shape[0] != batch:
        raise ValueError(f"shape mismatch: A {tuple(a.shape)} (a_mn={a_mn}) vs B {tuple(b.shape)} (b_mn={b_mn})")
    if out is None:
        out = torch.empty((batch, M, N), dtype=out_dtype, device=a.device)
        if a.dim() == 2:
            out = out[0]
    O = _as3d(out)
    if O.shape != (batch, M, N) or O.stride(-1) != 1:
        raise ValueError(f"bad output shape/stride {tuple(out.shape)}")
    if O.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("output must be bfloat16 or float32")
    CI = None
    if cin is not None:
        CI = _as3d(cin)
        if CI.shape != (batch, M, N) or CI.stride(-1) != 1 or CI.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("bad cin")
    f = _lib.fn("sr_gemm_bf16", _ARGTYPES)
    rc = f(A.data_ptr(), B.data_ptr(), O.data_ptr(), _lib.ptr(CI), M, N, K, batch,
           A.stride(1), B.stride(1), O.stride(1), CI.stride(1) if CI is not None else 0,
           A.stride(0), B.stride(0), O.stride(0), CI.stride(0) if CI is not None else 0,
           int(a_mn), int(b_mn), int(O.dtype == torch.float32),
           int(CI is not None and CI.dtype == torch.float32),
           float(alpha), float(beta), _lib.ptr(alpha_t), _lib.ptr(row_scale), int(sym), int(bn), int(max_ctas),
           _lib.status_buffer(a.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "sr_gemm_bf16")
    return out


FP8_DTYPES = {torch.float8_e4m3fn: 0, torch.float8_e5m2: 1}
_ARGTYPES_FP8 = _ARGTYPES[:16] + [_lib.c_int] * 4 + [_lib.c_float, _lib.c_float, _lib.c_void_p, _lib.c_void_p,
                                                     _lib.c_int, _lib.c_int, _lib.c_void_p, _lib.c_void_p]


def fp8_empty(shape, dtype, device) -> torch.Tensor:
    """Uninitialised 2-D fp8 tensor whose row stride is a multiple of 16 bytes (what a TMA operand needs); the view
    returned has exactly `shape`."""
    rows, cols = shape
    ld = (cols + 15) // 16 * 16
    return torch.empty((rows, ld), dtype=dtype, device=device)[:, :cols]


def quantize_fp8(x: torch.Tensor, scale: float, transpose: bool = False, dtype=torch.float8_e4m3fn) -> torch.Tensor:
    """fp8(x / scale) of a bf16 matrix [R, C] (saturating); `transpose` returns the [C, R] layout. Per-tensor static
    scales as in the reference's fp8 head (tiny/cuda_kernels.py:340-343)."""
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1:
        raise TypeError("quantize_fp8 expects a 2-D bf16 tensor with a contiguous last dimension")
    R, C = x.shape
    out = fp8_empty((C, R) if transpose else (R, C), dtype, x.device)
    if not x.is_cuda:
        src = (x.float() / scale).clamp(-torch.finfo(dtype).max, torch.finfo(dtype).max).to(dtype)
        out.copy_(src.t() if transpose else src)
        return out
    rc = _lib.fn("sr_quant_fp8", [_lib.c_void_p, _lib.c_void_p, ctypes.c_long, _lib.c_int, ctypes.c_long, ctypes.c_long,
                                  _lib.c_float, _lib.c_int, _lib.c_int, _lib.c_void_p])(
        x.data_ptr(), out.data_ptr(), R, C, x.stride(0), out.stride(0), float(scale), int(transpose),
        FP8_DTYPES[dtype], _lib.stream_ptr())
    _lib.check_rc(rc, "sr_quant_fp8")
    return out


def gemm_fp8(a, b, out=None, cin=None, *, alpha=1.0, beta=0.0, alpha_t=None, row_scale=None, out_dtype=torch.bfloat16,
             bn=0, max_ctas=0):
    """alpha * a @ b.T with fp8 operands a [.., M, K], b [.., N, K] (K contiguous, K % 16 == 0) on the CTA-pair
    tcgen05 kernel with kind::f8f6f4 MMAs and fp32 accumulation. The scales of a per-tensor quantisation go into
    alpha. The reference calls torch._scaled_mm (cuBLASLt) for these products (tiny/cuda_kernels.py:345-352)."""
    if a.dtype not in FP8_DTYPES or b.dtype not in FP8_DTYPES:
        raise TypeError("gemm_fp8 operands must be float8_e4m3fn or float8_e5m2")
    A, B = _as3d(a), _as3d(b)
    batch, M, K = A.shape
    N = B.shape[1]
    if B.shape[0] != batch or B.shape[2] != K or A.stride(-1) != 1 or B.stride(-1) != 1:
        raise ValueError(f"shape mismatch: {tuple(a.shape)} vs {tuple(b.shape)}")
    if out is None:
        out = torch.empty((batch, M, N), dtype=out_dtype, device=a.device)
        if a.dim() == 2:
            out = out[0]
    O = _as3d(out)
    CI = _as3d(cin) if cin is not None else None
    f = _lib.fn("sr_gemm_fp8_pair", _ARGTYPES_FP8)
    rc = f(A.data_ptr(), B.data_ptr(), O.data_ptr(), _lib.ptr(CI), M, N, K, batch,
           A.stride(1), B.stride(1), O.stride(1), CI.stride(1) if CI is not None else 0,
           A.stride(0), B.stride(0), O.stride(0), CI.stride(0) if CI is not None else 0,
           FP8_DTYPES[a.dtype], FP8_DTYPES[b.dtype], int(O.dtype == torch.float32),
           int(CI is not None and CI.dtype == torch.float32), float(alpha), float(beta), _lib.ptr(alpha_t),
           _lib.ptr(row_scale), int(bn), int(max_ctas), _lib.status_buffer(a.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "sr_gemm_fp8_pair")
    return out


def mm_nt(x, w, **kw):
    """x[M,K] @ w[N,K].T"""
    return gemm(x, w, **kw)


def mm_nn(x, w, **kw):
    """x[M,K] @ w[K,N]"""
    return gemm(x, w, b_mn=True, **kw)


def mm_tn(x, y, **kw):
    """x[K,M].T @ y[K,N]"""
    return gemm(x, y, a_mn=True, b_mn=True, **kw)


def set_pair_mode(on: bool) -> None:
    """Route eligible products to the CTA-pair kernel (`csrc/gemm_tcgen05_pair.cu`, the default) or keep every
    product on the single-CTA kernel. `SR_GEMM_PAIR=0` in the environment selects the latter at import."""
    f = _lib.lib().sr_gemm_set_pair_mode
    f.argtypes = [_lib.c_int]
    f.restype = None
    f(1 if on else 0)
