"""The NumPy oracle against golden vectors produced by the reference interpreter (tests/golden/).

Bit-exact wherever NumPy evaluates the same expression tree; the one float32 matmul case differs
from the interpreter only in BLAS blocking and is held to 1e-5.
"""

from __future__ import annotations

import hashlib

import numpy as np
import pytest
from conftest import BF16, F16, F32, bits, load_golden

from enceladus_b200.workloads import zipf_clipped


def same(a, b):
    np.testing.assert_array_equal(bits(a), bits(b))


def test_softmax(oracle):
    g = load_golden("softmax")
    keys = [k[:-2] for k in g if k.endswith("_x")]
    assert len(keys) == 6
    for k in keys:
        same(oracle.softmax(g[k + "_x"]), g[k + "_y"])
    x = np.random.default_rng(0).standard_normal((4096, 1024)).astype(np.float32) * 4
    y = oracle.softmax(x)
    digest = np.frombuffer(hashlib.sha256(y.tobytes()).digest(), np.uint8)
    same(digest, g["config1_sha256"])
    same(y[:8], g["config1_rows0_8"])


def test_layernorm(oracle):
    g = load_golden("layernorm")
    keys = [k[:-2] for k in g if k.endswith("_x")]
    assert len(keys) == 5
    for k in keys:
        block = int(k.rsplit("_b", 1)[1])
        y, mean, rstd = oracle.layernorm(g[k + "_x"], g[k + "_w"], g[k + "_b"], 1e-5, block)
        same(y, g[k + "_y"]), same(mean, g[k + "_mean"]), same(rstd, g[k + "_rstd"])


def test_rmsnorm(oracle):
    g = load_golden("rmsnorm")
    for k in [k[:-2] for k in g if k.endswith("_x")]:
        same(oracle.rmsnorm(g[k + "_x"], g[k + "_w"], 1e-6), g[k + "_y"])


def test_gelu(oracle):
    g = load_golden("gelu")
    for k in [k[:-2] for k in g if k.endswith("_x") and not k.startswith("tanh")]:
        same(oracle.fused_gelu(g[k + "_x"], g[k + "_bias"], 0.75), g[k + "_y"])
    same(oracle.gelu_tanh(g["tanh_f32_x"]), g["tanh_f32_y"])


def test_matmul(oracle):
    g = load_golden("matmul")
    for k in [k[:-2] for k in g if k.endswith("_a")]:
        if k.startswith("fused"):
            got = oracle.matmul_bias_gelu(g[k + "_a"], g[k + "_b"], g[k + "_bias"], 64 if "256x512" in k else 32)
        else:
            got = oracle.matmul(g[k + "_a"], g[k + "_b"], 32)
        if g[k + "_c"].dtype == F32:
            np.testing.assert_allclose(got, g[k + "_c"], rtol=1e-5, atol=1e-5)
        else:
            same(got, g[k + "_c"])


def test_int_matmul(oracle):
    """Integer tl.dot: int8, uint8, int16, int32 at full range (wraps modulo 2^32) and the sums float32 cannot hold."""
    g = load_golden("int_matmul")
    keys = [k[:-2] for k in g if k.endswith("_a")]
    assert len(keys) == 10
    for k in keys:
        same(oracle.int_matmul(g[k + "_a"], g[k + "_b"]), g[k + "_c"])


def attention_cases():
    g = load_golden("attention")
    i = 0
    while f"case{i}_meta" in g:
        n, d, causal, bm, bn, code = (int(v) for v in g[f"case{i}_meta"])
        dt = [F32, F16, BF16][code]
        r = np.random.default_rng(n + d)
        q, k, v = (r.standard_normal((2, 2, n, d)).astype(np.float32).astype(dt) for _ in range(3))
        yield i, q, k, v, bool(causal), (0.3 if causal else None), bm, bn, g[f"case{i}_o"]
        i += 1


def test_attention(oracle):
    count = 0
    for _, q, k, v, causal, scale, bm, bn, want in attention_cases():
        o, lse = oracle.attention(q, k, v, causal, scale, bm, bn, return_lse=True)
        same(o, want)
        # The logsumexp output has no counterpart in the reference: pin it to the float64 definition.
        np.testing.assert_allclose(lse, oracle.attention_lse_f64(q, k, v, causal, scale), atol=1e-4, rtol=0)
        count += 1
    assert count == 12


def test_attention_block_size_changes_only_last_bits(oracle):
    _, q, k, v, causal, scale, _, _, want = next(c for c in attention_cases() if c[0] == 10)
    o = oracle.attention(q, k, v, causal, scale, 128, 128)
    np.testing.assert_allclose(o.astype(np.float32), want.astype(np.float32), atol=2e-2, rtol=0)


def test_histogram(oracle):
    g = load_golden("histogram")
    x = np.random.default_rng(5).standard_normal(100_003).astype(np.float32)
    same(oracle.histogram(x, 48, -3.0, 3.0), g["f32_100003_48bins"])
    x = np.random.default_rng(0).integers(0, 256, 1 << 18).astype(np.int32)
    same(oracle.histogram(x, 256, 0.0, 256.0), g["i32_uniform256_2p18"])
    x = zipf_clipped(np.random.default_rng(1), 1 << 16, 1.1, 4096)
    same(oracle.histogram(x, 4096, 0.0, 4096.0), g["i32_zipf4096_2p16"])


CUMSUM_DTYPES = {"f32": F32, "f16": F16, "bf16": BF16, "int8": np.dtype(np.int8), "int64": np.dtype(np.int64),
                 "int32": np.dtype(np.int32)}


def cumsum_input(name: str, shape):
    dt = CUMSUM_DTYPES[name]
    r = np.random.default_rng(shape[1])
    if dt.kind in "iu":
        return r.integers(-100, 100, shape).astype(dt)
    return (r.standard_normal(shape) * 4).astype(np.float32).astype(dt)


def test_cumsum(oracle):
    g = load_golden("cumsum")
    seen = 0
    for k in g:
        if "_rev" not in k:
            continue
        name, shape, rev = k.split("_")
        shape = tuple(int(s) for s in shape.split("x"))
        same(oracle.cumsum(cumsum_input(name, shape), bool(int(rev[-1]))), g[k])
        seen += 1
    assert seen == 36
    x = np.random.default_rng(9).integers(0, 1 << 20, (2, 65536)).astype(np.int32)
    y = oracle.cumsum(x)
    same(y[:, -16:], g["i32_wrap_2x65536_tail"])
    same(np.frombuffer(hashlib.sha256(y.tobytes()).digest(), np.uint8), g["i32_wrap_2x65536_sha256"])
    assert (y[:, -1] < 0).any() or (np.diff(y.astype(np.int64), axis=1) < 0).any()  # the sums really wrap


@pytest.mark.parametrize("n", [1, 5, 4097])
def test_flat_cumsum_is_the_row_rule(oracle, n):
    x = np.random.default_rng(n).integers(0, 16, n).astype(np.int32)
    same(oracle.cumsum(x), oracle.cumsum(x[None, :])[0])
