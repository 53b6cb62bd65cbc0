"""The allocation-free column sum, called through its exported C symbol.

Some users of the kernel library may not allocate device memory at the point where they
need a bias gradient (inside stream capture, or when a host framework hands them nothing
but input and output pointers). ``nfn_colsum_noalloc`` serves them with scratch that is
compiled into the library. This test checks it against the ordinary entry point, twice in
a row, because the built-in scratch is shared and keeps the previous call's contents.
Collected last so that a failure here cannot hide results of the other tests.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, dy, out, accumulate=0):
    fn = lib.nfn_colsum_noalloc
    fn.restype = ctypes.c_int
    rows, C = dy.shape
    return fn(ctypes.c_void_p(dy.data_ptr()), ctypes.c_int(dy.stride(0)), ctypes.c_void_p(out.data_ptr()),
              ctypes.c_int(rows), ctypes.c_int(C), ctypes.c_int(accumulate),
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_noalloc_matches_scratch_version_twice(kernel_lib):
    from neuralfn_b200.ops import kernels as K
    torch.manual_seed(0)
    shapes = [(4096, 3072), (1000, 770)]          # the second call sees the first call's leftovers
    for rows, C in shapes:
        wide = torch.randn(rows, C + 62, device="cuda", dtype=torch.bfloat16)
        dy = wide[:, :C]                                     # row stride larger than the width
        want = torch.empty(C, device="cuda", dtype=torch.bfloat16)
        K.colsum(dy, want, torch.empty(64 * C, device="cuda", dtype=torch.float32))
        got = torch.full((C,), 7.0, device="cuda", dtype=torch.bfloat16)
        before = torch.cuda.memory_allocated()
        assert _call(kernel_lib, dy, got) == 0
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        ref = dy.float().sum(0)
        # both entry points add the same bf16 values in fp32, in different orders: equal up to the
        # final bf16 rounding
        assert ((got.float() - want.float()).norm() / want.float().norm()).item() < 5e-3
        assert ((got.float() - ref).norm() / ref.norm()).item() < 1e-2
    # accumulate on top of an existing gradient
    acc = want.clone()
    assert _call(kernel_lib, dy, acc, accumulate=1) == 0
    torch.cuda.synchronize()
    assert ((acc.float() - 2 * ref).norm() / (2 * ref).norm()).item() < 2e-2


def test_noalloc_rejects_oversize(kernel_lib):
    dy = torch.zeros(8, 8194, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(8194, device="cuda", dtype=torch.bfloat16)
    assert _call(kernel_lib, dy, out) != 0
    kernel_lib.nfn_last_error.restype = ctypes.c_char_p
    assert b"8192" in kernel_lib.nfn_last_error()


def test_noalloc_rejects_misaligned_view(kernel_lib):
    """A bf16 view that starts at an odd element has even sizes but a 2-byte aligned address; the
    entry point must refuse it on the host (no launch, so nothing can fault on the device)."""
    from neuralfn_b200.ops import _lib
    wide = torch.zeros(16, 66, device="cuda", dtype=torch.bfloat16)
    dy = wide[:, 1:65]
    assert dy.data_ptr() % 4 == 2 and dy.shape[1] % 2 == 0 and dy.stride(0) % 2 == 0
    out = torch.zeros(64, device="cuda", dtype=torch.bfloat16)
    before = _lib.launch_count()
    assert _call(kernel_lib, dy, out) != 0
    assert _lib.launch_count() == before
    kernel_lib.nfn_last_error.restype = ctypes.c_char_p
    assert b"aligned" in kernel_lib.nfn_last_error()
    torch.cuda.synchronize()
    _lib.assert_status_ok("colsum_noalloc misaligned")
