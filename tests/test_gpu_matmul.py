"""Parity of the tcgen05 matmul (and its CUDA-core fallback) with the oracle and the golden vectors."""

from __future__ import annotations

import numpy as np
import pytest
from conftest import BF16, F16, F32, assert_close, load_golden
from test_gpu_parity import host, torch_of

import enceladus_b200 as enceladus
from enceladus_b200 import _native as N
from enceladus_b200 import ops

pytestmark = pytest.mark.gpu


def operands(rng, m, n, k, dt):
    a = (rng.uniform(-1, 1, (m, k)) / np.sqrt(k)).astype(np.float32).astype(dt)
    b = (rng.uniform(-1, 1, (k, n)) / np.sqrt(k)).astype(np.float32).astype(dt)
    bias = (0.1 * rng.standard_normal(n)).astype(np.float32).astype(dt)
    return a, b, bias


def test_matmul_golden():
    g = load_golden("matmul")
    for k in [k[:-2] for k in g if k.endswith("_a")]:
        if k.startswith("fused"):
            got = ops.matmul_bias_gelu(g[k + "_a"], g[k + "_b"], g[k + "_bias"])
        else:
            got = ops.matmul_desc(g[k + "_a"], g[k + "_b"])
        want = g[k + "_c"]
        tol = 1e-4 * np.sqrt(g[k + "_a"].shape[1]) if want.dtype == F32 else None  # reference: tests/test_interpreter.py:87
        assert_close(got, want, atol=tol, rtol=tol, what=k)


@pytest.mark.parametrize("dt", [F16, BF16], ids=str)
@pytest.mark.parametrize("mnk", [(128, 256, 64), (128, 256, 128), (256, 512, 1024), (1024, 1024, 1024), (1000, 520, 264),
                                 (130, 72, 8), (64, 64, 64), (513, 520, 520), (2048, 256, 4096)], ids=str)
def test_fused_matmul_shapes(oracle, dt, mnk):
    m, n, k = mnk
    a, b, bias = operands(np.random.default_rng(m + n + k), m, n, k, dt)
    want = oracle.matmul_bias_gelu(a, b, bias, bk=64)
    got = host(ops.matmul_bias_gelu(torch_of(a), torch_of(b), torch_of(bias)))
    assert_close(got, want)
    plain = host(ops.matmul_desc(torch_of(a), torch_of(b)))
    assert_close(plain, oracle.matmul(a, b, 64))


def test_matmul_every_variant(oracle):
    from enceladus_b200.configs import MATMUL_TILES

    assert N.num_variants(N.K_MATMUL) == len(MATMUL_TILES)
    a, b, bias = operands(np.random.default_rng(0), 700, 900, 520, F16)
    want = oracle.matmul_bias_gelu(a, b, bias, bk=64)
    at, bt, biast = torch_of(a), torch_of(b), torch_of(bias)
    for v, (bm, bn, bk, _) in enumerate(MATMUL_TILES):
        assert f"tile=128x{bn}x64" in N.variant_info(N.K_MATMUL, v)
        c = enceladus.new_empty(at, (700, 900))
        grid = (enceladus.cdiv(900, bn), enceladus.cdiv(700, bm))
        ops.matmul_bias_gelu_kernel[grid](at, bt, biast, c, 700, 900, 520, 520, 900, 900, BM=bm, BN=bn, BK=bk, variant=v)
        assert_close(host(c), want, what=f"variant {v}")
    enceladus.synchronize()


def test_matmul_strided_views_and_unaligned_fallback(oracle):
    a, b, bias = operands(np.random.default_rng(1), 300, 400, 256, F16)
    big_a, big_b = torch_of(np.pad(a, ((0, 0), (0, 64)))), torch_of(np.pad(b, ((0, 0), (0, 112))))
    av, bv = big_a[:, :256], big_b[:, :400]  # leading dimensions 320 and 512
    want = oracle.matmul_bias_gelu(a, b, bias, bk=64)
    assert_close(host(ops.matmul_bias_gelu(av, bv, torch_of(bias))), want)
    a2, b2, bias2 = operands(np.random.default_rng(2), 100, 90, 70, BF16)  # leading dimensions 70 and 90: no TMA
    assert_close(host(ops.matmul_bias_gelu(torch_of(a2), torch_of(b2), torch_of(bias2))), oracle.matmul_bias_gelu(a2, b2, bias2, 32))


@pytest.mark.parametrize("dt", [F16, BF16], ids=str)
@pytest.mark.parametrize("mnk", [(513, 513, 513), (257, 130, 71), (129, 1000, 333), (64, 65, 2049), (1, 7, 9)], ids=str)
def test_matmul_operands_tma_cannot_describe(oracle, dt, mnk):
    """Odd leading dimensions (the reference's 513^3 shape among them) and bases that are not 16-byte aligned: the
    tensor-core kernel's loader warps fill the swizzled stages themselves; every tile variant, ragged edges in all
    three dimensions, fused and plain."""
    m, n, k = mnk
    a, b, bias = operands(np.random.default_rng(m * n + k), m, n, k, dt)
    want = oracle.matmul_bias_gelu(a, b, bias, bk=64)
    at, bt, biast = torch_of(a), torch_of(b), torch_of(bias)
    for v in [None, *range(N.num_variants(N.K_MATMUL))]:
        c = enceladus.new_empty(at, (m, n))
        ops.matmul_bias_gelu_kernel[(enceladus.cdiv(n, 64), enceladus.cdiv(m, 128))](at, bt, biast, c, m, n, k, k, n, n, BM=128, BN=64,
                                                                                   BK=64, variant=v)
        assert_close(host(c), want, what=f"variant {v}")
    assert_close(host(ops.matmul_desc(at, bt)), oracle.matmul(a, b, 64))
    # aligned leading dimensions but a base shifted by one element (2 bytes)
    import torch

    flat = torch.zeros(m * (k + 8) + 1, dtype=at.dtype, device="cuda")
    shifted = flat[1:].view(m, k + 8)[:, :k]
    shifted.copy_(at)
    assert_close(host(ops.matmul_bias_gelu(shifted, bt, biast)), want)
    enceladus.synchronize()


def test_matmul_config3_rows_sampled(oracle):
    """Full-size fused matmul (8192^3 fp16): a sample of rows against the oracle, all rows against linearity."""
    import torch

    m = n = k = 8192
    g = torch.Generator(device="cuda").manual_seed(3)
    a = ((torch.rand(m, k, device="cuda", generator=g) * 2 - 1) / 8192**0.5).half()
    b = ((torch.rand(k, n, device="cuda", generator=g) * 2 - 1) / 8192**0.5).half()
    bias = (0.1 * torch.randn(n, device="cuda", generator=g)).half()
    c = ops.matmul_bias_gelu(a, b, bias)
    rows = np.random.default_rng(3).choice(m, 48, replace=False)
    want = oracle.matmul_bias_gelu(host(a[rows]), host(b), host(bias), bk=64)
    assert_close(host(c[rows]), want)
    # plain product: (2A) @ B == 2 (A @ B) exactly wherever the float16 result is a normal number
    # (scaling by two is exact in the float32 accumulator and in every normal float16)
    p1, p2 = ops.matmul_desc(a, b), ops.matmul_desc(a * 2, b)
    normal = p1.abs() > 2.0**-13
    assert torch.equal(p2[normal], (p1 * 2)[normal])
    assert float(normal.float().mean()) > 0.9
    enceladus.synchronize()


def test_autotuned_matmul_picks_a_variant(oracle, tmp_path, monkeypatch):
    monkeypatch.setenv("ENCELADUS_CACHE_DIR", str(tmp_path))
    a, b, _ = operands(np.random.default_rng(4), 512, 512, 512, F16)
    got = host(ops.matmul_tuned(torch_of(a), torch_of(b)))
    assert_close(got, oracle.matmul(a, b, 64))
    assert list(tmp_path.rglob("*.json")), "the tuning result was not persisted"


# ---- integer matmul: exact, int32 accumulation that wraps modulo 2^32 ------------------------------------
def test_int_matmul_golden():
    g = load_golden("int_matmul")
    keys = [k[:-2] for k in g if k.endswith("_a")]
    assert len(keys) == 10
    for k in keys:
        a, b = g[k + "_a"], g[k + "_b"]
        for dev in (False, True):  # NumPy arguments and device tensors
            got = ops.int_matmul(torch_of(a), torch_of(b)) if dev else ops.int_matmul(a, b)
            np.testing.assert_array_equal(host(got), g[k + "_c"], err_msg=k)


@pytest.mark.parametrize("dt", [np.int8, np.uint8])
@pytest.mark.parametrize("mkn", [(512, 1024, 768), (300, 2000, 130), (128, 4096, 256), (1000, 144, 1040)])
def test_int8_matmul_on_tensor_cores_is_exact(oracle, dt, mkn):
    """Full-range 8-bit operands on the tcgen05 path (K and N multiples of 16), every tile variant, ragged edges."""
    m, k, n = mkn
    r = np.random.default_rng(m + k + n)
    info = np.iinfo(dt)
    a = r.integers(info.min, info.max, (m, k), dt, endpoint=True)
    b = r.integers(info.min, info.max, (k, n), dt, endpoint=True)
    want = oracle.int_matmul(a, b)
    at, bt = torch_of(a), torch_of(b)
    for variant in range(N.num_variants(N.K_MATMUL_INT)):
        c = enceladus.new_empty(at, (m, n), np.int32)
        ops.int8_matmul_kernel[(enceladus.cdiv(n, 128), enceladus.cdiv(m, 128))](at, bt, c, m, n, k, BM=128, BN=128, BK=128,
                                                                           variant=variant)
        np.testing.assert_array_equal(host(c), want, err_msg=f"variant {variant}")


def test_int_matmul_wraps_and_takes_unaligned_and_wide_types(oracle):
    r = np.random.default_rng(5)
    # sums beyond 2^31: int8 extremes over K = 2^17 wrap modulo 2^32 on the tensor-core path
    k = 1 << 17
    a, b = np.full((128, k), -128, np.int8), np.full((k, 16), -128, np.int8)
    np.testing.assert_array_equal(host(ops.int_matmul(torch_of(a), torch_of(b))), oracle.int_matmul(a, b))
    # shapes TMA cannot describe (odd leading dimensions) and 16/32-bit operands: CUDA cores, same result
    for dt, (m, kk, n) in ((np.int8, (50, 100, 33)), (np.uint8, (77, 45, 130)), (np.int16, (64, 200, 96)), (np.int32, (33, 70, 65))):
        info = np.iinfo(dt)
        a = r.integers(info.min, info.max, (m, kk), dt, endpoint=True)
        b = r.integers(info.min, info.max, (kk, n), dt, endpoint=True)
        np.testing.assert_array_equal(host(ops.int_matmul(torch_of(a), torch_of(b))), oracle.int_matmul(a, b), err_msg=str(dt))
    with pytest.raises(TypeError, match="int8, uint8, int16 or int32"):
        ops.int_matmul(torch_of(np.zeros((8, 8), np.float16)), torch_of(np.zeros((8, 8), np.float16)))
