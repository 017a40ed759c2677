"""Parity at the benchmark sizes themselves: 2^30-element histogram and int32 cumsum, 2^28-element float32
cumsum, the K = 16384 fused matmul, and LayerNorm rows that take the kernel's ill-conditioned branch.

The inputs of the 2^30 / 2^28 cases are generated on the device (seeded `torch.Generator`) and copied to
the host for the oracle, which walks them in chunks: histograms of chunks add, and the scan of a
concatenation is the scan of each chunk plus the wrapped total of the chunks before it, so the chunked
comparison is the same bit-exact statement as one call over the whole array
(np.cumsum rule: src/enceladus/language/ops.py:2047-2060; bin rule: examples/09_histogram.py:37-41).
"""

from __future__ import annotations

import math

import numpy as np
import pytest
from conftest import BF16, F16, F32, assert_close

import enceladus_b200 as enceladus
from enceladus_b200 import _native as N
from enceladus_b200 import ops

pytestmark = pytest.mark.gpu

CHUNK = 1 << 26


def torch_of(a: np.ndarray):
    from enceladus_b200.runtime import interop

    return interop._np_as_torch_view(np.ascontiguousarray(a)).to("cuda")


def host(t) -> np.ndarray:
    from enceladus_b200.testing import _host

    return _host(t)


def gen(seed: int):
    import torch

    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return g


def zipf_on_device(n: int, bins: int, seed: int):
    """Zipf(1.1) clipped to bins-1, sampled by inverse CDF on the truncated support (the law of
    enceladus_b200.workloads.zipf_clipped), in pieces of 2^26 so that the float64 uniforms stay small."""
    import torch
    from scipy.special import zeta

    kk = np.arange(1, bins - 1, dtype=np.float64)
    cdf = torch.from_numpy(np.concatenate([[0.0], np.cumsum(kk ** -1.1 / zeta(1.1, 1))])).cuda()
    x = torch.empty(n, device="cuda", dtype=torch.int32)
    g = gen(seed)
    for s0 in range(0, n, CHUNK):
        u = torch.rand(min(CHUNK, n - s0), device="cuda", generator=g, dtype=torch.float64)
        x[s0 : s0 + CHUNK] = torch.searchsorted(cdf, u, right=True).clamp_(max=bins - 1).int()
    return x


@pytest.mark.parametrize("kind,bins", [("uniform256", 256), ("zipf4096", 4096)])
def test_histogram_2p30_bit_exact(oracle, kind, bins):
    import torch

    n = 1 << 30
    if kind == "uniform256":
        x = torch.randint(0, 256, (n,), device="cuda", dtype=torch.int32, generator=gen(30))
    else:
        x = zipf_on_device(n, bins, 31)
    xh = x.cpu().numpy()
    want = np.zeros(bins, np.int64)
    for s0 in range(0, n, CHUNK):
        want += oracle.histogram(xh[s0 : s0 + CHUNK], bins, 0.0, float(bins))
    assert int(want.sum()) == n and int(want.max()) < 2**31  # every value is in range; no bin wraps int32
    want = want.astype(np.int32)
    for v in (None, N.num_variants(N.K_HISTOGRAM) - 1):
        hist = torch.zeros(bins, device="cuda", dtype=torch.int32)
        ops.histogram_kernel[(enceladus.cdiv(n, 1024),)](x, hist, n, 0.0, 1.0, NUM_BINS=bins, BLOCK=1024, variant=v)
        np.testing.assert_array_equal(host(hist), want, err_msg=f"{kind} variant {v}")
    enceladus.synchronize()


def test_cumsum_int32_2p30_bit_exact(oracle):
    """2^30 int32 values in [0, 16): byte offsets pass 2^32, 262144 ring tiles; the default (bulk-copy ring)
    variant and the widest register variant, both against np.cumsum chunk by chunk."""
    import torch

    n = 1 << 30
    x = torch.randint(0, 16, (n,), device="cuda", dtype=torch.int32, generator=gen(32))
    xh = x.cpu().numpy()
    out = torch.empty_like(x)
    for v in (None, 2):
        out.fill_(-1)
        ops.cumsum_kernel[(1,)](out, x, 1, n, n, n, REVERSE=False, BLOCK_M=1, BLOCK_N=1 << 30, variant=v)
        enceladus.synchronize()  # raises if a look-back wait ran out
        got = out.cpu().numpy()
        carry = np.uint32(0)
        for s0 in range(0, n, CHUNK):
            want = (oracle.cumsum(xh[s0 : s0 + CHUNK]).view(np.uint32) + carry).view(np.int32)
            np.testing.assert_array_equal(got[s0 : s0 + CHUNK], want, err_msg=f"variant {v} chunk at {s0}")
            carry = np.uint32(want.view(np.uint32)[-1])
        del got


def test_cumsum_int32_2p30_wraps(oracle):
    """The same length with values up to 2^28, so that the running sum wraps modulo 2^32 about every 32 elements."""
    import torch

    n = 1 << 30
    x = torch.randint(0, 1 << 28, (n,), device="cuda", dtype=torch.int32, generator=gen(33))
    xh = x.cpu().numpy()
    out = torch.empty_like(x)
    ops.cumsum_kernel[(1,)](out, x, 1, n, n, n, REVERSE=False, BLOCK_M=1, BLOCK_N=1 << 30)
    enceladus.synchronize()
    got = out.cpu().numpy()
    carry = np.uint32(0)
    for s0 in range(0, n, CHUNK):
        want = (oracle.cumsum(xh[s0 : s0 + CHUNK]).view(np.uint32) + carry).view(np.int32)
        np.testing.assert_array_equal(got[s0 : s0 + CHUNK], want, err_msg=f"chunk at {s0}")
        carry = np.uint32(want.view(np.uint32)[-1])


def test_cumsum_float32_2p28_tolerance(oracle):
    """2^28 N(0,1) values.  Bar: no further from the float64 scan than the reference's own sequential float32
    accumulation is, with 1e-4 of the largest exact prefix as the floor (the reference's relative bound,
    tests/test_atomics_scans.py:225)."""
    import torch

    n = 1 << 28
    x = torch.randn(n, device="cuda", generator=gen(34))
    xh = x.cpu().numpy()
    exact = np.cumsum(xh, dtype=np.float64)
    ref_err = float(np.abs(oracle.cumsum(xh).astype(np.float64) - exact).max())
    bound = max(ref_err, 1e-4 * float(np.abs(exact).max()))
    out = torch.empty_like(x)
    for v in (None, 2):
        out.fill_(0)
        ops.cumsum_kernel[(1,)](out, x, 1, n, n, n, REVERSE=False, BLOCK_M=1, BLOCK_N=1 << 28, variant=v)
        enceladus.synchronize()
        err = float(np.abs(out.cpu().numpy().astype(np.float64) - exact).max())
        assert err <= bound, (v, err, bound, ref_err)


def test_matmul_config3b_rows_sampled(oracle):
    """C = GELU(A @ B + bias) at M = N = 4096, K = 16384 (256 K-steps per tile): 48 sampled rows against the
    oracle's float32 accumulation in K blocks of 64, float16 tolerance (1e-3, 2e-3)."""
    m = n = 4096
    k = 16384
    r = np.random.default_rng(0)
    sc = np.float32(1 / math.sqrt(k))
    a = ((r.random((m, k), dtype=np.float32) * 2 - 1) * sc).astype(np.float16)
    b = ((r.random((k, n), dtype=np.float32) * 2 - 1) * sc).astype(np.float16)
    bias = (0.1 * r.standard_normal(n, dtype=np.float32)).astype(np.float16)
    got = host(ops.matmul_bias_gelu(torch_of(a), torch_of(b), torch_of(bias)))
    rows = np.concatenate([[0, 1, 127, 128, m - 1], r.integers(0, m, 43)])
    want = oracle.matmul_bias_gelu(a[rows], b, bias, 64)
    assert_close(got[rows], want)
    assert np.isfinite(got.astype(np.float32)).all()


# ---- LayerNorm rows whose mean is large against their spread ----------------------------------------------
# The kernel takes sum and sum of squares in one pass and switches to the centred second pass when
# mean^2 > 16 var.  The reference computes (x - mean) * rstd with mean rounded to float32 once
# (examples/03_layernorm.py:26-42), so its own y carries an error of about |mean| * 2^-24 * rstd; the kernel
# forms x * rstd - mean * rstd, which rounds once more at the same magnitude.  Bar, in units of the output:
#   |y - y_oracle| <= tol(dtype) + 4 * 2^-24 * |mean| * rstd * |w|
# i.e. the dtype tolerance of well-conditioned rows plus four float32 half-ulps of mean/sigma.
@pytest.mark.parametrize("dt", [F32, BF16, F16], ids=str)
@pytest.mark.parametrize("ratio", [8.0, 100.0])
def test_layernorm_large_mean_rows(oracle, dt, ratio):
    r = np.random.default_rng(int(ratio))
    m, n = 64, 4096
    x = (r.standard_normal((m, n)) + ratio).astype(np.float32).astype(dt)
    x[::7] = (r.standard_normal((len(x[::7]), n)) - ratio).astype(np.float32).astype(dt)  # negative means too
    w = (1 + 0.1 * r.standard_normal(n)).astype(np.float32).astype(dt)
    b = (0.1 * r.standard_normal(n)).astype(np.float32).astype(dt)
    y, mean, rstd = ops.layernorm(torch_of(x), torch_of(w), torch_of(b))
    wy, wm, wr = oracle.layernorm(x, w, b)
    # statistics: the centred branch must give the reference's variance, not E[x^2] - mean^2
    assert_close(host(mean), wm, atol=1e-5, rtol=1e-5)
    assert_close(host(rstd), wr, atol=1e-5, rtol=1e-5)
    atol, rtol = {F32: (1e-4, 1e-5), F16: (1e-3, 2e-3), BF16: (1e-2, 1.6e-2)}[dt]
    slack = 4 * 2.0**-24 * np.abs(wm * wr)[:, None] * np.abs(w.astype(np.float32))[None, :]
    diff = np.abs(host(y).astype(np.float64) - wy.astype(np.float64))
    assert (diff <= atol + rtol * np.abs(wy.astype(np.float64)) + slack).all(), float(diff.max())


@pytest.mark.parametrize("dt", [F32, BF16], ids=str)
def test_layernorm_constant_rows(oracle, dt):
    """var = 0: rstd = 1/sqrt(eps), y = b exactly where the row is constant (x - mean = 0)."""
    m, n = 9, 1024
    r = np.random.default_rng(5)
    x = np.repeat(r.standard_normal((m, 1)).astype(np.float32) * 3, n, axis=1).astype(dt)
    x[0] = 0
    w = (1 + 0.1 * r.standard_normal(n)).astype(np.float32).astype(dt)
    b = (0.1 * r.standard_normal(n)).astype(np.float32).astype(dt)
    y, mean, rstd = ops.layernorm(torch_of(x), torch_of(w), torch_of(b))
    wy, wm, wr = oracle.layernorm(x, w, b)
    assert_close(host(mean), wm, atol=1e-6, rtol=1e-6)
    # the reference's mean of n equal values can differ from the value by an ulp, which 1/sqrt(1e-5) = 316 amplifies;
    # rstd itself must agree, and y must stay within that amplified ulp of b
    assert_close(host(rstd), wr, atol=0, rtol=1e-4)
    amp = 316.3 * np.abs(x.astype(np.float32)).max() * 2.0**-23 * 1.2
    assert_close(host(y), wy, atol=amp + (1e-2 if dt == BF16 else 1e-5), rtol=1.6e-2 if dt == BF16 else 1e-5)


def test_layernorm_ill_conditioned_every_variant(oracle):
    """The vote that sends a whole CTA down the centred branch: CTAs that mix well- and ill-conditioned rows."""
    import torch

    r = np.random.default_rng(6)
    m, n = 96, 2048
    x = r.standard_normal((m, n)).astype(np.float32)
    x[1::3] += 50.0
    xb = x.astype(BF16)
    w, b = (1 + 0.1 * r.standard_normal(n)).astype(np.float32).astype(BF16), (0.1 * r.standard_normal(n)).astype(np.float32).astype(BF16)
    wy, wm, wr = oracle.layernorm(xb, w, b)
    xt, wt, bt = torch_of(xb), torch_of(w), torch_of(b)
    for v in range(N.num_variants(N.K_LAYERNORM)):
        y = enceladus.new_empty(xt)
        mean, rstd = torch.empty(m, device="cuda"), torch.empty(m, device="cuda")
        ops.layernorm_kernel[(m,)](xt, y, wt, bt, mean, rstd, n, n, n, 1e-5, BLOCK=1024, variant=v)
        assert_close(host(mean), wm, atol=1e-5, rtol=1e-5, what=f"mean variant {v}")
        assert_close(host(rstd), wr, atol=1e-5, rtol=1e-5, what=f"rstd variant {v}")
        assert_close(host(y), wy, what=f"variant {v}")
