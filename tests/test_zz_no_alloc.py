"""The allocation-free column-sum entry point, called through its exported C symbol.

Some embedders may not allocate device memory at all once they are running (a
server that owns the whole device through its own arena, a plug-in inside a host
with a fixed memory plan), so they cannot give ``mimir_colsum`` the scratch buffer
it asks for.  ``mimir_colsum_noalloc`` keeps that scratch inside the library.
This file checks it against ``mimir_colsum`` on two calls in a row (the calls
share the built-in scratch, so the second one must not see anything stale from
the first), and that oversized inputs are refused with a message.
The file name sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbols():
    from mimir_b200 import _native
    lib = _native.lib()
    fn = lib.mimir_colsum_noalloc  # resolved by name from the shared library
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_int, ctypes.c_void_p]
    return lib, fn


def test_noalloc_colsum_matches_colsum_twice_in_a_row():
    from mimir_b200.ops import kernels as K
    lib, fn = _symbols()
    stream = torch.cuda.current_stream().cuda_stream
    torch.manual_seed(11)
    # second shape is narrower and shorter than the first: stale partials would show
    for rows, N in ((4096, 3072), (700, 776)):
        x = torch.randn(rows, N, device="cuda").bfloat16()
        want = torch.empty(N, device="cuda", dtype=torch.bfloat16)
        K.colsum(x, want, torch.empty(64 * N, device="cuda"))
        got = torch.full((N,), 7.0, device="cuda", dtype=torch.bfloat16)
        # one warm-up call (the first call on a device looks up the scratch address), then the call
        # that is measured: the DRIVER's count of free bytes must not move, which also sees an
        # allocation made behind torch's back
        rc = fn(x.data_ptr(), rows, N, x.stride(0), got.data_ptr(), 0, stream)
        assert rc == 0, lib.mimir_last_error().decode()
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        rc = fn(x.data_ptr(), rows, N, x.stride(0), got.data_ptr(), 0, stream)
        assert rc == 0, lib.mimir_last_error().decode()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before
        ref = x.float().sum(0)
        tol = 2e-2 * (ref.abs().max().item() + 1e-3)
        assert torch.equal(got, want)            # same split and order of sums as mimir_colsum: same bits
        assert (got.float() - ref).abs().max().item() <= tol
        # accumulate on top of the previous result
        rc = fn(x.data_ptr(), rows, N, x.stride(0), got.data_ptr(), 1, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert (got.float() - 2 * ref).abs().max().item() <= 2 * tol + 2e-2 * ref.abs().max().item()


def test_noalloc_colsum_refuses_what_it_cannot_serve():
    lib, fn = _symbols()
    stream = torch.cuda.current_stream().cuda_stream
    x = torch.zeros(8, 16392, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(16392, device="cuda", dtype=torch.bfloat16)
    assert fn(x.data_ptr(), 8, 16392, 16392, out.data_ptr(), 0, stream) == -1
    assert b"exceeds" in lib.mimir_last_error()
    assert fn(x.data_ptr(), 8, 12, 16392, out.data_ptr(), 0, stream) == -1
    assert fn(x.data_ptr(), 8, 64, 32, out.data_ptr(), 0, stream) == -1       # row pitch below the width
    assert b"pitch" in lib.mimir_last_error()
