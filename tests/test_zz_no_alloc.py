"""The allocation-free Muon post-processing entry point, called through its exported C symbol.

Some users of the kernel library must not allocate device memory when they run this step (they sit inside another
framework's allocator hook or callback, or their process has given away all device memory up front), so
`sr_muon_post_noalloc` keeps its work arrays in a fixed device array inside the library. The test drives it with
ctypes exactly as such a caller would, twice in a row (the internal array keeps the previous call's contents, so the
second call proves nothing stale leaks through), in both the per-row and the per-column mode, and compares with the
ordinary entry point that takes caller-allocated work arrays. This file sorts last so that a run stopping at the
first failure has already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from slowrun_b200.ops import _lib as L
    lib = L.lib()
    lib.sr_muon_post_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                         ctypes.c_int, ctypes.c_float, ctypes.c_void_p]
    lib.sr_muon_post_noalloc.restype = ctypes.c_int
    lib.sr_muon_post_noalloc_max_elems.argtypes = []
    lib.sr_muon_post_noalloc_max_elems.restype = ctypes.c_long
    lib.sr_muon_post.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 3 + [ctypes.c_float, ctypes.c_void_p]
    lib.sr_muon_post.restype = ctypes.c_int
    return lib


def _reference(lib, X, S, beta2):
    n, r, c = X.shape
    ln = r if r >= c else c
    vmean = torch.empty(n, ln, device="cuda")
    fs = torch.empty(n, ln, device="cuda")
    U = torch.empty_like(X)
    rc = lib.sr_muon_post(X.data_ptr(), vmean.data_ptr(), S.data_ptr(), fs.data_ptr(), U.data_ptr(), n, r, c, beta2,
                          torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return U


def test_noalloc_entry_point_matches_regular_one_twice_in_a_row():
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    torch.manual_seed(0)
    beta2 = 0.94921875
    # first a column-mode problem, then a row-mode one of a different size: the second call sees the first one's
    # leftovers in the shared work array
    for (n, r, c) in [(3, 128, 640), (2, 512, 256), (3, 128, 640)]:
        X = (torch.randn(n, r, c, device="cuda") * 0.05).bfloat16()
        ln = r if r >= c else c
        S0 = torch.rand(n, ln, device="cuda") * 1e-3
        S_ref, S_new = S0.clone(), S0.clone()
        U_ref = _reference(lib, X, S_ref, beta2)
        U_new = torch.empty_like(X)
        before = torch.cuda.memory_allocated()
        rc = lib.sr_muon_post_noalloc(X.data_ptr(), S_new.data_ptr(), U_new.data_ptr(), n, r, c, beta2, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.allclose(S_new, S_ref, rtol=1e-4, atol=1e-9)
        err = (U_new.float() - U_ref.float()).abs().max().item()
        assert err <= 2e-2 * max(U_ref.float().abs().max().item(), 1e-6), err


def test_noalloc_entry_point_rejects_oversized_problems():
    lib = _lib()
    mx = lib.sr_muon_post_noalloc_max_elems()
    assert mx == 1 << 18
    n, r, c = 1, 8, mx + 4      # column mode: n * c exceeds the internal array
    X = torch.zeros(n, r, c, dtype=torch.bfloat16, device="cuda")
    S = torch.zeros(n, c, device="cuda")
    U = torch.empty_like(X)
    rc = lib.sr_muon_post_noalloc(X.data_ptr(), S.data_ptr(), U.data_ptr(), n, r, c, 0.95, torch.cuda.current_stream().cuda_stream)
    assert rc == -8
    torch.cuda.synchronize()


def test_noalloc_entry_point_at_exactly_the_limit_and_with_a_bad_column_count():
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    mx = lib.sr_muon_post_noalloc_max_elems()
    torch.manual_seed(1)
    n, r, c = 4, 64, mx // 4            # column mode, n * c == the limit exactly: accepted
    X = (torch.randn(n, r, c, device="cuda") * 0.05).bfloat16()
    S0 = torch.rand(n, c, device="cuda") * 1e-3
    S_ref, S_new = S0.clone(), S0.clone()
    U_ref = _reference(lib, X, S_ref, 0.94921875)
    U_new = torch.empty_like(X)
    assert lib.sr_muon_post_noalloc(X.data_ptr(), S_new.data_ptr(), U_new.data_ptr(), n, r, c, 0.94921875, stream) == 0
    torch.cuda.synchronize()
    assert torch.allclose(S_new, S_ref, rtol=1e-4, atol=1e-9)
    err = (U_new.float() - U_ref.float()).abs().max().item()
    assert err <= 2e-2 * max(U_ref.float().abs().max().item(), 1e-6), err
    # a column count that is not a multiple of four is refused before anything is launched
    Xb = torch.zeros(1, 8, 6, dtype=torch.bfloat16, device="cuda")
    Sb = torch.zeros(1, 8, device="cuda")
    assert lib.sr_muon_post_noalloc(Xb.data_ptr(), Sb.data_ptr(), torch.empty_like(Xb).data_ptr(), 1, 8, 6, 0.95, stream) == -2
    torch.cuda.synchronize()
