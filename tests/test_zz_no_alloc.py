"""The allocation-free C entry point (himuon_rmsnorm_bwd_noalloc) against the ordinary RMSNorm backward.

Some users of the library cannot allocate device memory at the call site: their host runtime owns all of it,
or they cannot take the implicit device synchronisation of cudaMalloc/cudaFree.  For them the library exports
one C function whose scratch is a fixed array inside the library image.  This test calls it the way such a
user would - through the exported C symbol with raw pointers - twice in a row with different inputs (the
second call must not see the first call's sums), and checks both results against the regular entry point.
It is collected last so that a run stopping at the first failure has already run every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from himuon_b200._build import so_path
    from himuon_b200._ext import ext

    ext()                                    # loads libtorch first so the shared object resolves
    lib = ctypes.CDLL(so_path())
    fn = lib.himuon_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.himuon_noalloc_last_error.restype = ctypes.c_char_p
    return lib, fn


def _reference(dy, x, w, rstd):
    from himuon_b200._ext import ext

    dx = torch.empty_like(x)
    acc = torch.zeros(x.shape[1], device="cuda", dtype=torch.float32)
    ext().rmsnorm_bwd(dy, x, w, rstd, dx, acc)
    return dx, acc.to(torch.bfloat16)


def test_no_alloc_entry_point_matches_regular_path_twice():
    from himuon_b200._ext import ext

    lib, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row with different shapes, then the kernel variants for wide rows (cols > 5120), the largest
    # supported width, and a narrow call after a wide one (the scratch still holds the wide call's sums)
    for seed, (rows, cols) in enumerate([(513, 2560), (300, 1024), (96, 8192), (40, 16384), (130, 512)]):
        torch.manual_seed(seed)
        x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
        w = (1 + 0.1 * torch.randn(cols, device="cuda")).bfloat16()
        dy = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
        y = torch.empty_like(x)
        rstd = torch.empty(rows, device="cuda", dtype=torch.float32)
        ext().rmsnorm_fwd(x, w, y, rstd, 1e-6)
        want_dx, want_dw = _reference(dy, x, w, rstd)
        dx = torch.empty_like(x)
        dw = torch.empty(cols, device="cuda", dtype=torch.bfloat16)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), rows, cols, stream)
        torch.cuda.synchronize()
        assert rc == 0, lib.himuon_noalloc_last_error().decode()
        assert torch.cuda.memory_allocated() == before
        assert torch.equal(dx, want_dx)
        err = (dw.float() - want_dw.float()).abs()
        assert (err <= 0.3 + 2e-2 * want_dw.float().abs()).all(), err.max()


def test_no_alloc_entry_point_rejects_oversized_input():
    lib, fn = _lib()
    t = torch.zeros(8, device="cuda", dtype=torch.bfloat16)
    f = torch.zeros(8, device="cuda", dtype=torch.float32)
    rc = fn(t.data_ptr(), t.data_ptr(), t.data_ptr(), f.data_ptr(), t.data_ptr(), t.data_ptr(), 1, 16384 + 8, 0)
    assert rc != 0 and b"exceeds" in lib.himuon_noalloc_last_error()


def test_no_alloc_entry_point_rejects_misaligned_pointers_on_the_host():
    lib, fn = _lib()
    rows, cols = 4, 64
    x = torch.zeros(rows * cols + 8, device="cuda", dtype=torch.bfloat16)
    f = torch.zeros(rows, device="cuda", dtype=torch.float32)
    good = x.data_ptr()
    bad = good + 2                        # one bf16 element off a 16-byte boundary
    assert good % 16 == 0
    for which in range(5):                # dy, x, w, dx, dw in turn
        ptrs = [good] * 5
        ptrs[which] = bad
        rc = fn(ptrs[0], ptrs[1], ptrs[2], f.data_ptr(), ptrs[3], ptrs[4], rows, cols, 0)
        assert rc != 0 and b"16-byte aligned" in lib.himuon_noalloc_last_error(), which
    torch.cuda.synchronize()              # nothing was launched, the context is untouched
