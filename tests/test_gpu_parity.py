"""Parity of the CUDA kernels with the oracle and with the reference-interpreter golden vectors.

Every launch goes through the public launch path (`kernel[grid](...)` -> registry -> ctypes -> C ABI).
Integer results must be bit-exact; float results use the reference's own differential-test tolerances
(tests/conftest.py:75-79 of the reference): fp32 (1e-5, 1e-5), fp16 (1e-3, 2e-3), bf16 (1e-2, 1.6e-2).
"""

from __future__ import annotations

import numpy as np
import pytest
from conftest import BF16, F16, F32, assert_close, load_golden

import enceladus_b200 as enceladus
from enceladus_b200 import _native as N
from enceladus_b200 import ops
from enceladus_b200.workloads import zipf_clipped

pytestmark = pytest.mark.gpu


def torch_of(a: np.ndarray):
    import torch

    from enceladus_b200.runtime import interop

    return interop._np_as_torch_view(np.ascontiguousarray(a)).to("cuda")


def host(t) -> np.ndarray:
    from enceladus_b200.testing import _host

    return _host(t)


def randn(rng, shape, dt):
    return rng.standard_normal(shape).astype(np.float32).astype(dt)


# ---- softmax ---------------------------------------------------------------------------------------
def test_softmax_golden():
    g = load_golden("softmax")
    for k in [k[:-2] for k in g if k.endswith("_x")]:
        assert_close(ops.softmax(g[k + "_x"]), g[k + "_y"], what=k)  # NumPy arguments: staged and copied back


def test_softmax_config1(oracle):
    x = np.random.default_rng(0).standard_normal((4096, 1024)).astype(np.float32) * 4
    want = oracle.softmax(x)
    got = host(ops.softmax(torch_of(x)))
    assert_close(got, want)
    assert_close(got[:8], load_golden("softmax")["config1_rows0_8"])
    np.testing.assert_allclose(got.sum(axis=1, dtype=np.float64), 1.0, atol=1e-5)


@pytest.mark.parametrize("dt", [F32, F16, BF16], ids=str)
@pytest.mark.parametrize("shape", [(1, 1), (5, 33), (64, 4096), (33, 5000), (3, 40_000), (2, 65_536)])
def test_softmax_shapes(oracle, dt, shape):
    x = randn(np.random.default_rng(shape[1]), shape, dt) * dt.type(4)
    assert_close(host(ops.softmax(torch_of(x))), oracle.softmax(x))


def test_softmax_strided_rows_and_offset_views(oracle):
    import torch

    x = randn(np.random.default_rng(1), (16, 1024), F32)
    big = torch_of(x)
    view = big[2:11, 4:1004]  # row stride 1024, 16-byte aligned start but ragged length
    assert_close(host(ops.softmax(view)), oracle.softmax(x[2:11, 4:1004]))
    odd = big[:, 1:1001]  # misaligned start: scalar path
    assert_close(host(ops.softmax(odd)), oracle.softmax(x[:, 1:1001]))
    full = torch.full((9, 2048), 7.0, device="cuda")
    out = full[:, :1000]  # strided output: the gaps between rows must stay untouched
    ops.softmax_kernel[(9,)](out, view, 1024, 2048, 1000, BLOCK=1024)
    assert_close(host(out), oracle.softmax(x[2:11, 4:1004]))
    assert float(full[:, 1000:].min()) == 7.0 and float(full[:, 1000:].max()) == 7.0


def test_softmax_every_variant(oracle):
    x = randn(np.random.default_rng(2), (300, 2048), F16)
    want = oracle.softmax(x)
    xt = torch_of(x)
    for v in range(N.num_variants(N.K_SOFTMAX)):
        out = enceladus.new_empty(xt)
        ops.softmax_kernel[(300,)](out, xt, 2048, 2048, 2048, BLOCK=2048, variant=v)
        assert_close(host(out), want, what=f"variant {v}")


# ---- layernorm / rmsnorm ---------------------------------------------------------------------------
def test_layernorm_golden():
    g = load_golden("layernorm")
    for k in [k[:-2] for k in g if k.endswith("_x")]:
        block = int(k.rsplit("_b", 1)[1])
        y, mean, rstd = ops.layernorm(g[k + "_x"], g[k + "_w"], g[k + "_b"], 1e-5, block)
        assert_close(y, g[k + "_y"], atol=1e-4 if y.dtype == F32 else None, what=k)
        assert_close(mean, g[k + "_mean"], atol=1e-5, rtol=1e-5)
        assert_close(rstd, g[k + "_rstd"], atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dt,shape", [(BF16, (2048, 4096)), (F16, (7, 1000)), (F32, (64, 8192)), (BF16, (3, 20_000)),
                                      (F32, (2, 33_000)), (BF16, (5, 17))], ids=str)
def test_layernorm_shapes(oracle, dt, shape):
    r = np.random.default_rng(shape[0])
    x = randn(r, shape, dt)
    w = (1 + 0.1 * r.standard_normal(shape[1])).astype(np.float32).astype(dt)
    b = (0.1 * r.standard_normal(shape[1])).astype(np.float32).astype(dt)
    y, mean, rstd = ops.layernorm(torch_of(x), torch_of(w), torch_of(b))
    wy, wm, wr = oracle.layernorm(x, w, b)
    assert_close(host(y), wy, atol=1e-4 if dt == F32 else None)
    assert_close(host(mean), wm, atol=1e-5, rtol=1e-5)
    assert_close(host(rstd), wr, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dt", [BF16, F16, F32], ids=str)
@pytest.mark.parametrize("shape", [(77, 4096), (77, 4088), (5, 2056), (3, 2048), (130, 1024), (9, 8192)], ids=str)
def test_rows_that_fill_their_threads_and_rows_that_do_not(oracle, dt, shape):
    """Rows that are exactly threads x vectors wide take the kernels' path without bounds tests and, when they span two
    warps, a CTA of their own; rows a vector or more short of that, and odd row counts, take the general path.  All
    three row kernels, every dtype, against the oracle."""
    r = np.random.default_rng(shape[0] * 31 + shape[1])
    x = randn(r, shape, dt)
    w = (1 + 0.1 * r.standard_normal(shape[1])).astype(np.float32).astype(dt)
    b = (0.1 * r.standard_normal(shape[1])).astype(np.float32).astype(dt)
    y, mean, rstd = ops.layernorm(torch_of(x), torch_of(w), torch_of(b))
    wy, wm, wr = oracle.layernorm(x, w, b)
    assert_close(host(y), wy, atol=1e-4 if dt == F32 else None, what="layernorm")
    assert_close(host(mean), wm, atol=1e-5, rtol=1e-5)
    assert_close(host(rstd), wr, atol=1e-5, rtol=1e-5)
    assert_close(host(ops.rmsnorm(torch_of(x), torch_of(w))), oracle.rmsnorm(x, w), what="rmsnorm")
    assert_close(host(ops.softmax(torch_of(x))), oracle.softmax(x), what="softmax")


def test_rmsnorm_golden():
    g = load_golden("rmsnorm")
    for k in [k[:-2] for k in g if k.endswith("_x")]:
        assert_close(ops.rmsnorm(g[k + "_x"], g[k + "_w"], 1e-6), g[k + "_y"], what=k)


@pytest.mark.parametrize("dt,shape", [(BF16, (2048, 4096)), (F16, (9, 1000)), (F32, (4, 128)), (BF16, (3, 40_000))],
                         ids=str)
def test_rmsnorm_shapes(oracle, dt, shape):
    r = np.random.default_rng(shape[1])
    x, w = randn(r, shape, dt), (1 + 0.1 * r.standard_normal(shape[1])).astype(np.float32).astype(dt)
    assert_close(host(ops.rmsnorm(torch_of(x), torch_of(w))), oracle.rmsnorm(x, w))


def test_norm_variants(oracle):
    r = np.random.default_rng(3)
    x, w, b = randn(r, (100, 4096), BF16), randn(r, 4096, BF16), randn(r, 4096, BF16)
    wy, _, _ = oracle.layernorm(x, w, b)
    wr = oracle.rmsnorm(x, w)
    xt, wt, bt = torch_of(x), torch_of(w), torch_of(b)
    import torch

    for v in range(N.num_variants(N.K_LAYERNORM)):
        y = enceladus.new_empty(xt)
        mean = torch.empty(100, device="cuda")
        rstd = torch.empty(100, device="cuda")
        ops.layernorm_kernel[(100,)](xt, y, wt, bt, mean, rstd, 4096, 4096, 4096, 1e-5, BLOCK=1024, variant=v)
        assert_close(host(y), wy, what=f"layernorm variant {v}")
        o = enceladus.new_empty(xt)
        ops.rmsnorm_kernel[(100,)](xt, wt, o, 4096, 4096, 4096, 1e-6, BLOCK=4096, variant=v)
        assert_close(host(o), wr, what=f"rmsnorm variant {v}")


# ---- GELU ------------------------------------------------------------------------------------------
def test_gelu_golden():
    g = load_golden("gelu")
    for k in [k[:-2] for k in g if k.endswith("_x") and not k.startswith("tanh")]:
        assert_close(ops.fused_gelu(g[k + "_x"], g[k + "_bias"], 0.75), g[k + "_y"], what=k)
    assert_close(ops.tanh_gelu(g["tanh_f32_x"]), g["tanh_f32_y"])


@pytest.mark.parametrize("n", [1, 3, 1023, (1 << 20) + 3])
def test_tanh_gelu_sizes_and_variants(oracle, n):
    x = (np.random.default_rng(n).standard_normal(n) * 2).astype(np.float32)
    want = oracle.gelu_tanh(x)
    xt = torch_of(x)
    for v in [None, *range(N.num_variants(N.K_GELU))]:
        out = enceladus.new_empty(xt)
        ops.tanh_gelu_kernel[(enceladus.cdiv(n, 1024),)](xt, out, n, BLOCK=1024, variant=v)
        assert_close(host(out), want, what=f"variant {v}")


def test_fused_gelu_ragged_columns_and_misaligned_base(oracle):
    r = np.random.default_rng(4)
    x, bias = randn(r, (257, 301), BF16), randn(r, 301, BF16)
    assert_close(host(ops.fused_gelu(torch_of(x), torch_of(bias), 1.5)), oracle.fused_gelu(x, bias, 1.5))
    flat = torch_of(randn(r, 4099, F32))
    xs = flat[3:]  # 12-byte offset
    out = enceladus.new_empty(xs)
    ops.tanh_gelu_kernel[(5,)](xs, out, 4096, BLOCK=1024)
    assert_close(host(out), oracle.gelu_tanh(host(xs)))


def test_add(oracle):
    r = np.random.default_rng(5)
    for dt in (F32, F16, BF16):
        for n in (1, 1000, (1 << 16) + 3):
            x, y = randn(r, n, dt), randn(r, n, dt)
            assert_close(host(ops.add(torch_of(x), torch_of(y))), oracle.vector_add(x, y))


# ---- histogram -------------------------------------------------------------------------------------
def test_histogram_golden():
    g = load_golden("histogram")
    x = np.random.default_rng(5).standard_normal(100_003).astype(np.float32)
    np.testing.assert_array_equal(ops.histogram(x, 48, -3.0, 3.0), g["f32_100003_48bins"])
    x = np.random.default_rng(0).integers(0, 256, 1 << 18).astype(np.int32)
    np.testing.assert_array_equal(ops.histogram(x, 256, 0.0, 256.0), g["i32_uniform256_2p18"])
    x = zipf_clipped(np.random.default_rng(1), 1 << 16, 1.1, 4096)
    np.testing.assert_array_equal(ops.histogram(x, 4096, 0.0, 4096.0), g["i32_zipf4096_2p16"])


def test_histogram_int32_every_variant(oracle):
    n = (1 << 24) + 5
    u = np.random.default_rng(0).integers(0, 256, n).astype(np.int32)
    z = zipf_clipped(np.random.default_rng(1), n, 1.1, 4096)
    wu, wz = oracle.histogram(u, 256, 0.0, 256.0), oracle.histogram(z, 4096, 0.0, 4096.0)
    ut, zt = torch_of(u), torch_of(z)
    for v in range(N.num_variants(N.K_HISTOGRAM)):
        for xt, bins, want in ((ut, 256, wu), (zt, 4096, wz)):
            hist = enceladus.new_zeros(xt, (bins,), np.int32)
            ops.histogram_kernel[(enceladus.cdiv(n, 1024),)](xt, hist, n, 0.0, 1.0, NUM_BINS=bins, BLOCK=1024,
                                                             variant=v)
            np.testing.assert_array_equal(host(hist), want, err_msg=f"variant {v} bins {bins}")


def test_histogram_drops_out_of_range_nan_and_accumulates(oracle):
    x = np.array([-1.0, 0.0, 0.5, 3.999, 4.0, np.nan, np.inf, -np.inf, 1e30, 2.0], np.float32)
    want = oracle.histogram(x, 4, 0.0, 4.0)
    np.testing.assert_array_equal(ops.histogram(x, 4, 0.0, 4.0), want)
    big = np.array([-5, 0, 3, 4, 2**31 - 1, -(2**31), 2], np.int32)
    np.testing.assert_array_equal(ops.histogram(big, 4, 0.0, 4.0), oracle.histogram(big, 4, 0.0, 4.0))
    xt = torch_of(x)
    hist = enceladus.new_zeros(xt, (4,), np.int32)
    for _ in range(2):  # atomic_add semantics: a second launch adds to the first
        ops.histogram_kernel[(1,)](xt, hist, x.size, 0.0, 1.0, NUM_BINS=4, BLOCK=1024)
    np.testing.assert_array_equal(host(hist), 2 * want)


def test_histogram_misaligned_halfs_and_many_bins(oracle):
    r = np.random.default_rng(6)
    x = randn(r, 100_001, F16)
    xt = torch_of(x)[1:]
    np.testing.assert_array_equal(host(ops.histogram(xt, 64, -4.0, 4.0)), oracle.histogram(x[1:], 64, -4.0, 4.0))
    xb = randn(r, 50_000, BF16)
    np.testing.assert_array_equal(host(ops.histogram(torch_of(xb), 33, -2.0, 2.0)), oracle.histogram(xb, 33, -2.0, 2.0))
    big = r.integers(0, 100_000, 1 << 20).astype(np.int32)  # more bins than shared memory holds
    np.testing.assert_array_equal(host(ops.histogram(torch_of(big), 100_000, 0.0, 100_000.0)),
                                  oracle.histogram(big, 100_000, 0.0, 100_000.0))


# ---- cumsum ----------------------------------------------------------------------------------------
def test_cumsum_golden():
    from test_oracle_golden import cumsum_input

    g = load_golden("cumsum")
    for k in g:
        if "_rev" not in k:
            continue
        name, shape, rev = k.split("_")
        shape = tuple(int(s) for s in shape.split("x"))
        got = ops.cumsum(cumsum_input(name, shape), reverse=bool(int(rev[-1])))
        assert_close(got, g[k], atol=1e-4 if got.dtype == F32 else None, rtol=1e-4 if got.dtype == F32 else None, what=k)
    x = np.random.default_rng(9).integers(0, 1 << 20, (2, 65536)).astype(np.int32)
    np.testing.assert_array_equal(ops.cumsum(x)[:, -16:], g["i32_wrap_2x65536_tail"])


@pytest.mark.parametrize("n", [1, 7, 4096, 4097, 12_345, (1 << 24) + 13])
def test_flat_cumsum_int32_bit_exact(oracle, n):
    x = np.random.default_rng(n).integers(0, 1 << 28, n).astype(np.int32)  # wraps after ~16 elements
    want = oracle.cumsum(x)
    xt = torch_of(x)
    for v in [None, *range(N.num_variants(N.K_CUMSUM))]:
        out = enceladus.new_empty(xt)
        ops.cumsum_kernel[(1,)](out, xt, 1, n, n, n, REVERSE=False, BLOCK_M=1, BLOCK_N=enceladus.next_power_of_2(n),
                                variant=v)
        np.testing.assert_array_equal(host(out), want, err_msg=f"variant {v}")
    enceladus.synchronize()  # raises if a look-back wait ran out


def test_flat_cumsum_float32_tolerance(oracle):
    n = 1 << 24
    x = np.random.default_rng(0).standard_normal(n).astype(np.float32)
    exact = np.cumsum(x.astype(np.float64))
    ref_err = np.abs(oracle.cumsum(x).astype(np.float64) - exact).max()
    got = host(ops.cumsum(torch_of(x))).astype(np.float64)
    # no worse than the reference's own sequential float32 accumulation, floor 1e-4 of the range
    assert np.abs(got - exact).max() <= max(ref_err, 1e-4 * np.abs(exact).max())


def test_flat_cumsum_misaligned_and_other_dtypes(oracle):
    r = np.random.default_rng(7)
    x = r.integers(-100, 100, 50_001).astype(np.int32)
    xt = torch_of(x)[1:]
    np.testing.assert_array_equal(host(ops.cumsum(xt)), oracle.cumsum(x[1:]))
    for dt in (np.int8, np.int16, np.uint8, np.int64):
        v = r.integers(0, 100, 30_000).astype(dt)
        got = host(ops.cumsum(torch_of(v)))
        want = oracle.cumsum(v)
        np.testing.assert_array_equal(got, want.astype(got.dtype))
    for dt in (F16, BF16):
        v = randn(r, 20_000, dt)
        assert_close(host(ops.cumsum(torch_of(v))), oracle.cumsum(v), atol=0.5, rtol=2e-2)


def test_row_cumsum_shapes(oracle):
    r = np.random.default_rng(8)
    for shape in ((4096, 512), (3, 70_000), (1000, 7)):
        x = r.integers(-1000, 1000, shape).astype(np.int32)
        for rev in (False, True):
            np.testing.assert_array_equal(host(ops.cumsum(torch_of(x), reverse=rev)), oracle.cumsum(x, rev))
    import torch

    x = r.standard_normal((64, 1024)).astype(np.float32)
    view = torch_of(x)[:, 8:1000]  # strided rows
    assert_close(host(ops.cumsum(view)), oracle.cumsum(x[:, 8:1000]), atol=1e-3, rtol=1e-4)
    assert isinstance(view, torch.Tensor)


def test_sharded_flat_cumsum_matches_single_pass(oracle):
    """The multi-GPU recipe (local total -> offset -> seeded scan) on one device, shard by shard."""
    import torch

    from enceladus_b200 import dist as edist

    n, world = 1_000_003, 4
    x = np.random.default_rng(11).integers(0, 1 << 29, n).astype(np.int32)
    want = oracle.cumsum(x)
    shards = [torch_of(x[slice(*edist.shard_range(n, r, world, 4))]) for r in range(world)]
    gathered = torch.cat([edist.cuda_total(s) for s in shards])  # what the all-gather leaves on every rank
    offs = edist.exclusive_offsets(host(gathered))
    seeds = [edist.cuda_offset(gathered, r) for r in range(world)]  # one-thread kernel, stays on the stream
    np.testing.assert_array_equal(np.concatenate([host(t) for t in seeds]), offs)
    got = np.concatenate([host(edist.cuda_scan(s, seeds[r])) for r, s in enumerate(shards)])
    np.testing.assert_array_equal(got, want)
    # float32 totals are added in shard order, as the host rule does
    f = torch.tensor([0.1, 0.2, 0.3, 1e8], device="cuda")
    np.testing.assert_array_equal(np.concatenate([host(edist.cuda_offset(f, r)) for r in range(4)]),
                                  edist.exclusive_offsets(host(f)))


def test_enc_sum_matches_the_wrapped_total_for_every_dtype_and_alignment(oracle):
    import torch

    r = np.random.default_rng(14)
    for dt, lo, hi in ((np.int32, 0, 1 << 30), (np.int8, -128, 128), (np.uint8, 0, 256), (np.int16, -30000, 30000)):
        for n, off in ((1, 0), (1_000_003, 0), (70_001, 1), ((1 << 22) + 5, 3)):
            x = r.integers(lo, hi, n + off).astype(dt)
            xt = torch_of(x)[off:]  # off > 0: not 16-byte aligned, scalar path
            want = x[off:].astype(np.int64).sum() & 0xFFFFFFFF
            assert int(host(edist_total(xt))[0]) & 0xFFFFFFFF == want, (dt, n, off)
    xf = r.standard_normal(3_000_001).astype(np.float32)
    got = float(host(edist_total(torch_of(xf)))[0])
    assert abs(got - xf.astype(np.float64).sum()) <= 1e-3 * np.abs(xf).sum() ** 0.5 + 1e-2


def edist_total(t):
    from enceladus_b200 import dist as edist

    return edist.cuda_total(t)


def test_captured_scan_survives_a_larger_eager_scan(oracle):
    """A CUDA graph keeps the address of the scan's descriptor buffer.  A later eager scan that needs a larger
    buffer must not free or move the captured one: replaying the graph afterwards gives the same result."""
    import torch

    n_small = 300_007
    x = torch_of(np.random.default_rng(15).integers(0, 1 << 28, n_small).astype(np.int32))
    out = torch.empty_like(x)

    def scan():
        ops.cumsum_kernel[(1,)](out, x, 1, n_small, n_small, n_small, REVERSE=False, BLOCK_M=1, BLOCK_N=1 << 19)

    scan()  # sizes the per-device capture buffer; nothing can be allocated during capture
    torch.cuda.synchronize()
    want = oracle.cumsum(host(x))
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        scan()
    g.replay()
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host(out), want)
    # 6e8 int8 values -> 146k tiles of 4096 -> more than the 1 MiB of descriptors the buffer starts with
    n_big = 600_000_000
    big = torch.randint(0, 100, (n_big,), device="cuda", dtype=torch.int8)
    big_out = torch.empty(n_big, device="cuda", dtype=torch.int32)
    ops.cumsum_kernel[(1,)](big_out, big, 1, n_big, n_big, n_big, REVERSE=False, BLOCK_M=1, BLOCK_N=1 << 30)
    torch.cuda.synchronize()
    assert (int(big_out[-1]) & 0xFFFFFFFF) == (int(big.sum(dtype=torch.int64)) & 0xFFFFFFFF)
    del big, big_out
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host(out), want)
    enceladus.synchronize()


# ---- launch path -----------------------------------------------------------------------------------
def test_numpy_arguments_are_written_back_and_async_numpy_defers(oracle):
    x = np.random.default_rng(12).standard_normal((8, 256)).astype(np.float32)
    out = np.zeros_like(x)
    with enceladus.async_numpy(True):
        ops.softmax_kernel[(8,)](out, x, 256, 256, 256, BLOCK=256)
        enceladus.synchronize()
    assert_close(out, oracle.softmax(x))
    assert ops.softmax_kernel.last_launch["h2d_bytes"] == x.nbytes  # the dense output is not copied in


def test_piecewise_staging_of_numpy_arguments_gives_the_single_piece_result(monkeypatch):
    """Large NumPy launches are staged, run and copied back piece by piece on side streams.  The pieces are
    independent rows / elements / M-blocks / (batch, head) slices, so the result must be bit-identical to
    the one-piece launch on device tensors; thresholds are lowered so that small arrays take the path."""
    from enceladus_b200.runtime import jit

    monkeypatch.setattr(jit, "PIPELINE_MIN_BYTES", 1)
    monkeypatch.setattr(jit, "PIPELINE_PIECE_BYTES", 64 << 10)
    r = np.random.default_rng(21)

    def same(kernel, got, want, pieces_at_least=2):
        got, want = (got if isinstance(got, tuple) else (got,)), (want if isinstance(want, tuple) else (want,))
        assert kernel.last_launch.get("pieces", 0) >= pieces_at_least, kernel.last_launch
        for g, w in zip(got, want):
            assert isinstance(g, np.ndarray)
            np.testing.assert_array_equal(g.view(np.uint8), host(w).view(np.uint8))

    x = randn(r, (1000, 520), F32)                       # ragged row count, rows not a multiple of 256 bytes
    same(ops.softmax_kernel, ops.softmax(x), ops.softmax(torch_of(x)))
    xb, w, b = randn(r, (777, 1024), BF16), randn(r, (1024,), BF16), randn(r, (1024,), BF16)
    same(ops.layernorm_kernel, ops.layernorm(xb, w, b), ops.layernorm(torch_of(xb), torch_of(w), torch_of(b)))
    same(ops.rmsnorm_kernel, ops.rmsnorm(xb, w), ops.rmsnorm(torch_of(xb), torch_of(w)))
    v = randn(r, (300001,), F32)
    same(ops.tanh_gelu_kernel, ops.tanh_gelu(v), ops.tanh_gelu(torch_of(v)))
    xg, bg = randn(r, (900, 200), F16), randn(r, (200,), F16)
    same(ops.fused_gelu_kernel, ops.fused_gelu(xg, bg, 0.5), ops.fused_gelu(torch_of(xg), torch_of(bg), 0.5))
    same(ops.add_kernel, ops.add(v, v[::-1].copy()), ops.add(torch_of(v), torch_of(v[::-1].copy())))
    a, bm, bias = randn(r, (600, 256), F16), randn(r, (256, 512), F16), randn(r, (512,), F16)
    same(ops.matmul_bias_gelu_kernel, ops.matmul_bias_gelu(a, bm, bias), ops.matmul_bias_gelu(torch_of(a), torch_of(bm), torch_of(bias)))
    q, k, vv = (randn(r, (2, 3, 256, 64), F16) for _ in range(3))  # lse rows of 1 KB keep every piece 256-byte aligned
    same(ops.attention_lse_kernel, ops.attention(q, k, vv, True, return_lse=True),
         ops.attention(torch_of(q), torch_of(k), torch_of(vv), True, return_lse=True))
    # the flat scan is cut along its one row; every piece is seeded with the last value of the piece before
    iv = r.integers(-2**31, 2**31, 200003, dtype=np.int64).astype(np.int32)   # wraps modulo 2^32 many times
    same(ops.cumsum_kernel, ops.cumsum(iv), ops.cumsum(torch_of(iv)))
    np.testing.assert_array_equal(ops.cumsum(iv), np.cumsum(iv.astype(np.int64)).astype(np.int32))
    big = r.integers(-2**31, 2**31, 500009, dtype=np.int64).astype(np.int32)  # a 2 MB output is page-locked: copied out per piece
    same(ops.cumsum_kernel, ops.cumsum(big), ops.cumsum(torch_of(big)))
    fv = randn(r, (150001,), F32)
    got = ops.cumsum(fv)
    assert ops.cumsum_kernel.last_launch.get("pieces", 0) >= 2
    exact = np.cumsum(fv.astype(np.float64))
    assert np.abs(got - exact).max() <= max(np.abs(np.cumsum(fv) - exact).max(), 1e-4 * np.abs(exact).max())
    ops.cumsum(fv, reverse=True)                                # suffix sums are not chained
    assert "pieces" not in ops.cumsum_kernel.last_launch
    # an array whose flat view is not a view (strided rows) takes the one-piece path
    xs = randn(r, (512, 1024), F32)[:, :512]
    got = ops.softmax(xs)
    assert "pieces" not in ops.softmax_kernel.last_launch
    np.testing.assert_array_equal(got, host(ops.softmax(torch_of(np.ascontiguousarray(xs)))))
    # ... and so does a strided NumPy output, whose gaps between rows must stay untouched
    full = np.full((9, 2048), 7.0, np.float32)
    ops.softmax_kernel[(9,)](full[:, :1000], xs[2:11, 4:504], 1024, 2048, 500, BLOCK=512)
    np.testing.assert_array_equal(full[:, :500], host(ops.softmax(torch_of(np.ascontiguousarray(xs[2:11, 4:504])))))
    assert full[:, 500:].min() == 7.0 and full[:, 500:].max() == 7.0


def test_injected_failure_surfaces_as_cuda_error():
    x = torch_of(np.zeros((2, 8), np.float32))
    N.load().enc_test_fail_next(N.ERR_LAUNCH)
    with pytest.raises(enceladus.CudaError, match="injected"):
        ops.softmax(x)
    ops.softmax(x)  # the next launch is unaffected
    enceladus.synchronize()


def test_bounded_device_wait_surfaces_at_synchronize_and_the_context_survives(oracle):
    """A device-side wait that runs out (a flag nothing sets, 2000 polls of 1 us) must not hang: the kernel
    returns, the next synchronize raises, and later launches work."""
    import torch

    stream = torch.cuda.current_stream().cuda_stream
    N.call("enc_test_device_wait", 2000, stream)
    with pytest.raises(enceladus.CudaError, match="device-side wait") as info:
        enceladus.synchronize()
    assert info.value.status == N.ERR_DEVICE_WAIT
    enceladus.synchronize()  # the status word was cleared by the report
    x = np.random.default_rng(13).standard_normal((4, 64)).astype(np.float32)
    assert_close(host(ops.softmax(torch_of(x))), oracle.softmax(x))
    with pytest.raises(ValueError, match="polls"):
        N.call("enc_test_device_wait", 2_000_000, stream)


def test_device_info_reports_blackwell():
    info = N.device_info()
    assert info.sm_count > 0 and info.cc_major >= 10, (info.cc_major, info.cc_minor)
