"""The reference interpreter itself as the checker, run at test time.

`oracle/_ref/` holds an install of the reference's CPU path (oracle/build_ref.py; built by
`__graft_entry__.build()` wherever a checkout exists).  These tests run its interpreter
(ENCELADUS_INTERPRET=1) on fresh seeded inputs - not the committed golden vectors - and hold to it
  * the NumPy restatement `oracle/enceladus_oracle.py`, bit for bit (CPU, no GPU needed), and
  * the CUDA kernels (marker `gpu`), with the reference's own tolerances.
They skip when nothing is installed.
"""

from __future__ import annotations

import numpy as np
import pytest
from conftest import BF16, F16, F32, assert_close

from oracle import ref_runtime

ref = ref_runtime.load()
pytestmark = pytest.mark.skipif(ref is None, reason="oracle/_ref is not installed (python oracle/build_ref.py)")


def randn(rng, shape, dt):
    return rng.standard_normal(shape).astype(np.float32).astype(dt)


def cases(seed: int):
    """name -> (interpreter result, arguments) on inputs drawn from `seed`."""
    r = np.random.default_rng(seed)
    x32 = randn(r, (33, 1000), F32) * np.float32(4)
    xb, w, b = randn(r, (17, 4096), BF16), randn(r, 4096, BF16), randn(r, 4096, BF16)
    xh, wh = randn(r, (9, 520), F16), randn(r, 520, F16)
    a, bm, bias = randn(r, (130, 96), F16), randn(r, (96, 200), F16), randn(r, 200, F16)
    q, k, v = (randn(r, (1, 2, 100, 64), F16) for _ in range(3))
    hx = randn(r, 50_000, F32)
    ci = r.integers(-1000, 1000, (5, 1000)).astype(np.int32)
    return {
        "softmax": (lambda: ref.example("02_softmax").softmax(x32), (x32,)),
        "layernorm": (lambda: ref.example("03_layernorm").layernorm(xb, w, b, 1e-5), (xb, w, b)),
        "rmsnorm": (lambda: ref.example("06_rmsnorm").rmsnorm(xh, wh, 1e-6), (xh, wh)),
        "fused_gelu": (lambda: ref.example("05_fused_gelu").fused_gelu(xh, wh, 0.75), (xh, wh)),
        "matmul_bias_gelu": (lambda: ref.example("07_matmul_fused").matmul_bias_gelu(a, bm, bias, bm=64, bn=64, bk=32), (a, bm, bias)),
        "attention": (lambda: ref.example("08_flash_attention").attention(q, k, v, True, block_m=64, block_n=64), (q, k, v)),
        "histogram": (lambda: ref.example("09_histogram").histogram(hx, 48, -3.0, 3.0), (hx,)),
        "cumsum": (lambda: ref.example("10_cumsum").cumsum(ci), (ci,)),
    }


def test_restatement_equals_the_live_interpreter(oracle):
    c = cases(101)
    same = np.testing.assert_array_equal
    same(oracle.softmax(*c["softmax"][1]), c["softmax"][0]())
    for got, want in zip(oracle.layernorm(*c["layernorm"][1], 1e-5), c["layernorm"][0]()):
        same(np.asarray(got).view(np.uint8), np.asarray(want).view(np.uint8))
    same(oracle.rmsnorm(*c["rmsnorm"][1], 1e-6), c["rmsnorm"][0]())
    same(oracle.fused_gelu(*c["fused_gelu"][1], 0.75), c["fused_gelu"][0]())
    same(oracle.matmul_bias_gelu(*c["matmul_bias_gelu"][1], 32), c["matmul_bias_gelu"][0]())
    same(oracle.attention(*c["attention"][1], True, None, 64, 64), c["attention"][0]())
    same(oracle.histogram(*c["histogram"][1], 48, -3.0, 3.0), c["histogram"][0]())
    same(oracle.cumsum(*c["cumsum"][1]), c["cumsum"][0]())


@pytest.mark.gpu
def test_cuda_kernels_against_the_live_interpreter():
    from enceladus_b200 import ops

    c = cases(202)
    assert_close(ops.softmax(*c["softmax"][1]), c["softmax"][0]())
    y, mean, rstd = ops.layernorm(*c["layernorm"][1], 1e-5)
    wy, wm, wr = c["layernorm"][0]()
    assert_close(y, wy)
    assert_close(mean, wm, atol=1e-5, rtol=1e-5)
    assert_close(rstd, wr, atol=1e-5, rtol=1e-5)
    assert_close(ops.rmsnorm(*c["rmsnorm"][1], 1e-6), c["rmsnorm"][0]())
    assert_close(ops.fused_gelu(*c["fused_gelu"][1], 0.75), c["fused_gelu"][0]())
    assert_close(ops.matmul_bias_gelu(*c["matmul_bias_gelu"][1]), c["matmul_bias_gelu"][0]())
    assert_close(ops.attention(*c["attention"][1], True), c["attention"][0](), atol=2e-3, rtol=2e-3)  # tests/test_attention.py:48
    np.testing.assert_array_equal(ops.histogram(*c["histogram"][1], 48, -3.0, 3.0), c["histogram"][0]())
    np.testing.assert_array_equal(ops.cumsum(*c["cumsum"][1]), c["cumsum"][0]())
