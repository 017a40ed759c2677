"""Parity of the flash-attention forward kernels (tcgen05 and CUDA-core) with the oracle and golden vectors."""

from __future__ import annotations

import numpy as np
import pytest
from conftest import BF16, F16, F32, assert_close
from test_gpu_parity import host, torch_of
from test_oracle_golden import attention_cases

import enceladus_b200 as enceladus
from enceladus_b200 import _native as N
from enceladus_b200 import ops

pytestmark = pytest.mark.gpu

# the reference's own tolerances for this kernel (tests/test_attention.py:48)
ATOL = {F16: 2e-3, F32: 1e-5, BF16: 2e-2}


def test_attention_golden(oracle):
    """The twelve reference test cases: outputs against the interpreter's, LSE against the oracle's."""
    seen = 0
    for i, q, k, v, causal, scale, bm, bn, want in attention_cases():
        o, lse = ops.attention(torch_of(q), torch_of(k), torch_of(v), causal, scale, return_lse=True)
        assert_close(host(o), want, atol=ATOL[want.dtype], what=f"case {i}")
        _, want_lse = oracle.attention(q, k, v, causal, scale, bm, bn, return_lse=True)
        np.testing.assert_allclose(host(lse), want_lse, atol=1e-3, rtol=0, err_msg=f"lse case {i}")
        seen += 1
    assert seen == 12


@pytest.mark.parametrize("dt", [BF16, F16], ids=str)
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(1, 2, 128, 128), (1, 3, 256, 128), (2, 2, 1000, 128), (1, 2, 1024, 64), (1, 1, 129, 128),
                                   (1, 2, 2048, 128)], ids=str)
def test_attention_shapes(oracle, dt, causal, shape):
    r = np.random.default_rng(shape[2] + shape[3])
    q, k, v = (r.standard_normal(shape).astype(np.float32).astype(dt) for _ in range(3))
    want, want_lse = oracle.attention(q, k, v, causal, None, 128, 128, return_lse=True)
    o, lse = ops.attention(torch_of(q), torch_of(k), torch_of(v), causal, return_lse=True)
    assert_close(host(o), want, atol=ATOL[dt])
    np.testing.assert_allclose(host(lse), want_lse, atol=1e-3, rtol=0)
    enceladus.synchronize()


def test_attention_large_scores_exercise_the_rescale(oracle):
    """Scores spread over many powers of two, so the running maximum keeps growing along the keys."""
    r = np.random.default_rng(0)
    shape = (1, 2, 512, 128)
    q = (r.standard_normal(shape) * 3).astype(np.float32).astype(BF16)
    k = (r.standard_normal(shape) * np.linspace(0.2, 3.0, 512)[None, None, :, None]).astype(np.float32).astype(BF16)
    v = r.standard_normal(shape).astype(np.float32).astype(BF16)
    for causal in (False, True):
        want, want_lse = oracle.attention(q, k, v, causal, 0.5, 128, 128, return_lse=True)
        o, lse = ops.attention(torch_of(q), torch_of(k), torch_of(v), causal, 0.5, return_lse=True)
        assert_close(host(o), want, atol=ATOL[BF16])
        np.testing.assert_allclose(host(lse), want_lse, atol=2e-3, rtol=1e-5)


def test_attention_every_variant_and_fallback(oracle):
    r = np.random.default_rng(1)
    q, k, v = (r.standard_normal((1, 2, 300, 128)).astype(np.float32).astype(F16) for _ in range(3))
    want = oracle.attention(q, k, v, True, None, 128, 128)
    qt, kt, vt = torch_of(q), torch_of(k), torch_of(v)
    for variant in range(N.num_variants(N.K_ATTENTION)):
        o = enceladus.new_empty(qt)
        ops.attention_kernel[(3, 2)](qt, kt, vt, o, 128**-0.5, 300, 300 * 128, 128, HEAD_DIM=128, BLOCK_M=128, BLOCK_N=128,
                                     CAUSAL=True, variant=variant)
        assert_close(host(o), want, atol=ATOL[F16], what=f"variant {variant}")
    for d, dt in ((16, F16), (32, BF16), (64, F32), (128, F32)):  # shapes the tensor-core kernel does not take
        q, k, v = (r.standard_normal((2, 1, 77, d)).astype(np.float32).astype(dt) for _ in range(3))
        for causal in (False, True):
            want, want_lse = oracle.attention(q, k, v, causal, None, 32, 32, return_lse=True)
            o, lse = ops.attention(torch_of(q), torch_of(k), torch_of(v), causal, return_lse=True)
            assert_close(host(o), want, atol=ATOL[dt] if dt != F32 else 2e-5)
            np.testing.assert_allclose(host(lse), want_lse, atol=1e-3, rtol=0)
    with pytest.raises(ValueError, match="head_dim"):
        ops.attention(torch_of(np.zeros((1, 1, 8, 48), np.float16)), torch_of(np.zeros((1, 1, 8, 48), np.float16)),
                      torch_of(np.zeros((1, 1, 8, 48), np.float16)))


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape,dt", [((4, 64, 512, 128), BF16), ((2, 50, 640, 128), F16), ((3, 70, 1000, 64), BF16),
                                      ((1, 160, 300, 128), F16)], ids=str)
def test_attention_many_items_per_cta(oracle, causal, shape, dt):
    """More work items (256 query rows of one (batch, head) slice) than SMs, so that every persistent CTA walks
    several items back to back: rings and barrier phases carry over from one item to the next, the last query
    block is ragged (640 rows: its second tile is empty; 1000 and 300 rows: partly filled), and with a causal
    mask the two tiles of an item need different numbers of key blocks.  Every variant must agree."""
    z, h, s_, d = shape
    r = np.random.default_rng(s_ + d + h)
    q, k, v = (r.standard_normal(shape).astype(np.float32).astype(dt) for _ in range(3))
    want, want_lse = oracle.attention(q, k, v, causal, None, 128, 128, return_lse=True)
    qt, kt, vt = torch_of(q), torch_of(k), torch_of(v)
    o, lse = ops.attention(qt, kt, vt, causal, return_lse=True)
    assert_close(host(o), want, atol=ATOL[dt])
    np.testing.assert_allclose(host(lse), want_lse, atol=1e-3, rtol=0)
    for variant in (3, 4):
        o2 = enceladus.new_empty(qt)
        ops.attention_kernel[(enceladus.cdiv(s_, 128), z * h)](qt, kt, vt, o2, d**-0.5, s_, s_ * d, d, HEAD_DIM=d, BLOCK_M=128,
                                                               BLOCK_N=128, CAUSAL=causal, variant=variant)
        assert_close(host(o2), want, atol=ATOL[dt], what=f"variant {variant}")
    enceladus.synchronize()  # raises if a bounded wait ran out


def test_attention_config4_slices_and_properties(oracle):
    """Full benchmark shape [8, 32, 4096, 128] bf16: two (batch, head) slices against the oracle, all of it
    against properties that hold for any size."""
    import torch

    g = torch.Generator(device="cuda").manual_seed(4)
    q, k, v = (torch.randn(8, 32, 4096, 128, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
    for causal in (False, True):
        o, lse = ops.attention(q, k, v, causal, return_lse=True)
        for b, h in ((0, 0), (7, 31)):
            sl = tuple(host(t[b : b + 1, h : h + 1]) for t in (q, k, v))
            want, want_lse = oracle.attention(*sl, causal, None, 128, 128, return_lse=True)
            assert_close(host(o[b : b + 1, h : h + 1]), want, atol=ATOL[BF16])
            np.testing.assert_allclose(host(lse[b : b + 1, h : h + 1]), want_lse, atol=1e-3, rtol=0)
        # a convex combination of the values: every output lies inside the range of V along the keys
        assert float(o.float().abs().max()) <= float(v.float().abs().max()) + 1e-2
        # values all equal to one: every output is one (the probabilities sum to one)
        ones = torch.ones_like(v)
        o1 = ops.attention(q, k, ones, causal)
        assert float((o1.float() - 1).abs().max()) < 1e-2
        if causal:  # the first query attends to the first key only
            assert torch.equal(o[:, :, 0], v[:, :, 0])
    enceladus.synchronize()
