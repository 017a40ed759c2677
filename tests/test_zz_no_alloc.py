"""The allocation-free flat scan (`enc_cumsum_noalloc`) against the ordinary entry point.

Some callers of the library may not allocate device memory at the moment they call it: a framework that
has given the whole device to its own memory pool, a serving loop that cannot take the stall of a
cudaMalloc, code that must not allocate after start-up.  For them the scan keeps its tile descriptors in a
fixed array inside the library instead of a buffer from cudaMalloc.  This file is collected last on
purpose: if it fails under `-x`, every other test has already run.

Both entry points are called through the C ABI (ctypes) on raw device pointers; the result of the new one
must equal the existing one's (integers bit for bit, float32 within the tolerance the other scan tests
use), on two calls in a row, because the array keeps the previous call's contents and must be cleared.
The integer results are also held to the oracle (np.cumsum in int32, wrapping modulo 2^32), so that the
two entry points cannot agree on a wrong answer.
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest

from enceladus_b200 import _native as N

pytestmark = pytest.mark.gpu


def _scan_both(x):
    """(result of enc_cumsum, result of enc_cumsum_noalloc, status word) for a flat device tensor."""
    import torch

    lib = N.load()
    stream = torch.cuda.current_stream().cuda_stream
    n = x.numel()
    code = {torch.int32: N.I32, torch.float32: N.F32}[x.dtype]
    ref, got = torch.empty_like(x), torch.empty_like(x)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    N.check(lib.enc_cumsum(x.data_ptr(), ref.data_ptr(), 1, n, n, n, 0, code, None, -1, stream))
    N.check(lib.enc_cumsum_noalloc(x.data_ptr(), got.data_ptr(), n, code, None, status.data_ptr(), stream))
    torch.cuda.synchronize()
    return ref, got, int(status.item())


def test_noalloc_scan_matches_the_allocating_entry_point_twice_in_a_row(oracle):
    import torch

    g = torch.Generator(device="cuda").manual_seed(0)
    # two different lengths and contents back to back: stale descriptors from the first call would
    # corrupt the second (the second is shorter, so part of the array is not even re-cleared by it)
    for n in ((1 << 22) + 12_345, (1 << 20) + 7):
        x = torch.randint(0, 1 << 28, (n,), device="cuda", dtype=torch.int32, generator=g)  # wraps mod 2^32
        ref, got, status = _scan_both(x)
        assert status == 0
        assert torch.equal(ref, got)
        np.testing.assert_array_equal(got.cpu().numpy(), oracle.cumsum(x.cpu().numpy()))
    for n in (3_000_001, 70_000):
        x = torch.randn(n, device="cuda", generator=g)
        ref, got, status = _scan_both(x)
        assert status == 0
        exact = np.cumsum(x.cpu().numpy().astype(np.float64))
        scale = max(np.abs(exact).max(), 1.0)
        # the same bound the float32 scan test uses: 1e-4 of the range, against the float64 scan
        assert np.abs(got.cpu().numpy() - exact).max() <= 1e-4 * scale
        assert np.abs(got.cpu().numpy() - ref.cpu().numpy()).max() <= 1e-4 * scale


def test_noalloc_scan_takes_a_seed_and_refuses_what_does_not_fit(oracle):
    import torch

    lib = N.load()
    stream = torch.cuda.current_stream().cuda_stream
    x = torch.randint(0, 9, (100_000,), device="cuda", dtype=torch.int32)  # small values: no wrap in this check
    seed = torch.tensor([41], device="cuda", dtype=torch.int32)
    out = torch.empty_like(x)
    N.check(lib.enc_cumsum_noalloc(x.data_ptr(), out.data_ptr(), x.numel(), N.I32, seed.data_ptr(), None, stream))
    torch.cuda.synchronize()
    want = torch.cumsum(x.to(torch.int64), 0) + 41
    assert torch.equal(out.to(torch.int64), want)
    # a seed that makes the very first output wrap: (2^31 - 1) + x[0] + ... in uint32 arithmetic
    seed = torch.tensor([2**31 - 1], device="cuda", dtype=torch.int32)
    N.check(lib.enc_cumsum_noalloc(x.data_ptr(), out.data_ptr(), x.numel(), N.I32, seed.data_ptr(), None, stream))
    torch.cuda.synchronize()
    want = (oracle.cumsum(x.cpu().numpy()).view(np.uint32) + np.uint32(2**31 - 1)).view(np.int32)
    np.testing.assert_array_equal(out.cpu().numpy(), want)
    too_long = (1 << 30) + 1  # refused before anything is touched, so the pointers are never read
    rc = lib.enc_cumsum_noalloc(ctypes.c_void_p(256), ctypes.c_void_p(256), too_long, N.I32, None, None, stream)
    assert rc == N.ERR_UNSUPPORTED and "exceed" in N.last_error()
    rc = lib.enc_cumsum_noalloc(x.data_ptr(), out.data_ptr(), 16, N.I64, None, None, stream)
    assert rc == N.ERR_UNSUPPORTED and "dtype" in N.last_error()
