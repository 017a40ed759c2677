"""Host-side launch path without a GPU: binding, grids, the registry, interop helpers, the autotuner's
selection rule and persistence, and the multi-GPU helpers (two gloo ranks on CPU)."""

from __future__ import annotations

import json
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np
import pytest

import enceladus_b200 as enceladus
import enceladus_b200.language as tl
from enceladus_b200 import dist as edist
from enceladus_b200.runtime import autotuner, jit, registry

ROOT = Path(__file__).resolve().parents[1]


def test_cdiv_and_next_power_of_2():
    assert [enceladus.cdiv(a, b) for a, b in ((0, 4), (1, 4), (4, 4), (5, 4))] == [0, 1, 1, 2]
    assert [enceladus.next_power_of_2(n) for n in (0, 1, 2, 3, 1000, 1024, 1025)] == [1, 1, 2, 4, 1024, 1024, 2048]


def test_signature_splits_constexpr_parameters():
    from enceladus_b200 import ops

    k = ops.softmax_kernel
    assert [p.name for p in k.params if p.is_constexpr] == ["BLOCK"]
    assert k.arg_names == ["out_ptr", "in_ptr", "stride_in", "stride_out", "n_cols", "BLOCK"]
    bound = k.bind((1, 2, 3, 4, 5), {"BLOCK": tl.constexpr(8)})
    assert bound["n_cols"] == 5 and bound["BLOCK"] == 8
    with pytest.raises(TypeError, match="softmax_kernel"):
        k.bind((1, 2), {})


def test_grid_forms():
    assert jit.resolve_grid((3,), {}) == (3, 1, 1)
    assert jit.resolve_grid(5, {}) == (5, 1, 1)
    assert jit.resolve_grid(lambda meta: (meta["n"] // 2, 2), {"n": 8}) == (4, 2, 1)
    with pytest.raises(ValueError, match="1 to 3 dimensions"):
        jit.resolve_grid((1, 2, 3, 4), {})
    with pytest.raises(ValueError, match="negative"):
        jit.resolve_grid((-1,), {})
    with pytest.raises(ValueError, match="limit"):
        jit.resolve_grid((1, 70000), {})


def test_calling_a_kernel_directly_is_an_error():
    from enceladus_b200 import ops

    with pytest.raises(RuntimeError, match=r"softmax_kernel\[grid\]"):
        ops.softmax_kernel(1, 2)


def test_zero_grid_is_a_silent_no_op():
    from enceladus_b200 import ops

    x = np.zeros((0, 8), np.float32)
    assert ops.softmax(x).shape == (0, 8)  # grid (0,) returns before touching the device


def test_unknown_kernel_has_no_fallback():
    @enceladus.jit
    def my_kernel(x_ptr, n, BLOCK: tl.constexpr):
        pass

    with pytest.raises(NotImplementedError, match="no code generator and no CPU fallback"):
        my_kernel[(1,)](np.zeros(4, np.float32), 4, BLOCK=4)

    @enceladus.jit
    def softmax_kernel(a, b):
        pass

    with pytest.raises(NotImplementedError, match="is known with parameters"):
        softmax_kernel[(1,)](1, 2)


def test_interpreter_request_is_refused(monkeypatch):
    from enceladus_b200 import ops

    monkeypatch.setenv("ENCELADUS_INTERPRET", "1")
    with pytest.raises(RuntimeError, match="not part of this build"):
        ops.softmax(np.zeros((2, 4), np.float32))


def test_launch_options_are_validated():
    from enceladus_b200 import ops

    x = np.zeros((2, 4), np.float32)
    with pytest.raises(ValueError, match="num_warps"):
        ops.softmax_kernel[(2,)](x, x, 4, 4, 4, BLOCK=4, num_warps=3)
    with pytest.raises(ValueError, match="dot_backend"):
        ops.softmax_kernel[(2,)](x, x, 4, 4, 4, BLOCK=4, dot_backend="cuda")
    with pytest.raises(TypeError, match=r"\*args"):
        enceladus.jit(lambda *a: None)


def test_registry_covers_the_kernel_set():
    want = {"softmax_kernel", "layernorm_kernel", "rmsnorm_kernel", "fused_gelu_kernel", "tanh_gelu_kernel",
            "matmul_bias_gelu_kernel", "matmul_desc_kernel", "matmul_kernel", "attention_kernel",
            "attention_lse_kernel", "histogram_kernel", "cumsum_kernel", "add_kernel"}
    assert want <= set(registry.kernels())
    from enceladus_b200 import ops

    for name in want - {"matmul_kernel"}:
        k = getattr(ops, name)
        assert registry.lookup(name, tuple(k.arg_names)).params == tuple(k.arg_names)


def test_interop_helpers_on_numpy():
    import ml_dtypes

    x = np.zeros((4, 10), np.float16)[:, ::2]
    assert enceladus.element_strides(x) == (10, 2)
    assert enceladus.element_dtype(x) == np.float16
    y = enceladus.new_empty(x, (3,), np.float32)
    assert isinstance(y, np.ndarray) and y.shape == (3,) and y.dtype == np.float32
    z = enceladus.new_zeros(np.zeros(2, ml_dtypes.bfloat16))
    assert z.dtype == ml_dtypes.bfloat16 and not z.astype(np.float32).any()
    with pytest.raises(TypeError, match="supported array type"):
        enceladus.element_strides([1, 2])


def test_interop_helpers_on_torch_cpu_tensors():
    import torch

    t = torch.zeros(4, 6, dtype=torch.bfloat16)[:, :3]
    assert enceladus.element_strides(t) == (6, 1)
    assert str(enceladus.element_dtype(t)) == "bfloat16"
    out = enceladus.new_zeros(t, (5,), np.int32)
    assert out.dtype == torch.int32 and out.shape == (5,)
    from enceladus_b200 import ops

    with pytest.raises(TypeError, match="CUDA tensor"):
        ops.softmax(torch.zeros(2, 4))


def test_read_only_numpy_output_is_refused(monkeypatch):
    import torch

    from enceladus_b200.runtime import interop

    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    st = interop.Staged()
    a = np.zeros(4, np.float32)
    a.flags.writeable = False
    with pytest.raises(ValueError, match="read-only"):
        st.to_device("out_ptr", a, written=True)
    with pytest.raises(ValueError, match="negative stride"):
        st.to_device("x", np.zeros(4, np.float32)[::-1], written=False)


def test_config_round_trip_and_identity():
    c = enceladus.Config({"BM": 128, "BN": 256, "BK": 64}, num_warps=8, dot_warps=[4, 2], variant=2)
    assert c.dot_warps == (4, 2)
    d = enceladus.Config.from_json(json.loads(json.dumps(c.to_json())))
    assert d == c and d.tag() == c.tag()
    assert c.launch_options() == {"num_warps": 8, "dot_warps": (4, 2), "variant": 2}
    assert "variant=2" in str(c)
    with pytest.raises(ValueError, match="dot_backend"):
        enceladus.Config({}, dot_backend="cuda")


def test_configs_lists():
    from enceladus_b200 import configs

    mm = configs.matmul_configs("float16")
    assert [c.variant for c in mm] == list(range(len(mm))) and all({"BM", "BN", "BK"} <= set(c.kwargs) for c in mm)
    assert configs.matmul_configs(np.float32) and configs.matmul_configs(tl.bfloat16)
    with pytest.raises(ValueError, match="matmul_configs supports"):
        configs.matmul_configs("int8")
    at = configs.attention_configs("bfloat16", 128)
    assert all({"BLOCK_M", "BLOCK_N"} <= set(c.kwargs) for c in at)
    with pytest.raises(ValueError, match="head dimensions"):
        configs.attention_configs("float16", 48)


def _tuner(monkeypatch, tmp_path, times, tolerance=0.01):
    """An autotuner over a stand-in kernel whose per-variant launch time is scripted by `times` (milliseconds)."""
    monkeypatch.setenv("ENCELADUS_CACHE_DIR", str(tmp_path))

    @enceladus.jit
    def add_kernel(x_ptr, y_ptr, out_ptr, n, BLOCK: tl.constexpr):
        pass

    calls = []
    monkeypatch.setattr(add_kernel, "run", lambda *a, grid, **kw: calls.append(kw.get("variant")))
    configs = [enceladus.Config({"BLOCK": 256 << i}, variant=i) for i in range(len(times))]
    state = {"current": None}

    def scripted(launch, count):  # stands in for the CUDA-event timer: runs the launches, reports the script's time
        out = []
        for _ in range(count):
            launch()
            out.append(times[calls[-1]])
        return out

    monkeypatch.setattr(autotuner, "time_launches", scripted)
    monkeypatch.setattr(autotuner, "on_device", lambda v: v)
    monkeypatch.setattr(autotuner, "device_tag", lambda: "test-arch")
    tuned = enceladus.autotune(configs=configs, key=["n"], tolerance=tolerance, warmup_ms=0)(add_kernel)
    return tuned, calls, configs, state


def test_autotuner_earliest_within_tolerance_wins(monkeypatch, tmp_path):
    tuned, calls, configs, _ = _tuner(monkeypatch, tmp_path, [1.000, 0.995, 2.0])
    x = np.zeros(8, np.float32)
    tuned[(1,)](x, x, x, 8)
    assert tuned.config_for(x, x, x, 8) is configs[0]  # 0.5% slower than the fastest, but earlier
    assert calls[-1] == 0
    n_calls = len(calls)
    tuned[(1,)](x, x, x, 8)
    assert len(calls) == n_calls + 1  # the second launch does not re-tune


def test_autotuner_picks_the_fastest_outside_tolerance_and_persists(monkeypatch, tmp_path):
    tuned, calls, configs, _ = _tuner(monkeypatch, tmp_path, [1.0, 0.5, 2.0])
    x = np.zeros(8, np.float32)
    tuned[(1,)](x, x, x, 8)
    assert tuned.config_for(x, x, x, 8) is configs[1]
    files = list(Path(tmp_path).rglob("test-arch.json"))
    assert len(files) == 1
    saved = json.loads(files[0].read_text())
    assert next(iter(saved["results"].values()))["config"]["variant"] == 1 and "library" in saved
    # a new tuner for the same kernel reads the file and does not benchmark
    tuned2, calls2, configs2, _ = _tuner(monkeypatch, tmp_path, [9.0, 9.0, 9.0])
    tuned2[(1,)](x, x, x, 8)
    assert calls2 == [1]
    # a new key (different n or dtype) tunes again
    y = np.zeros(16, np.float32)
    tuned2[(1,)](y, y, y, 16)
    assert len(calls2) > 2
    # a saved winner is an index into the library's variant list: another list (another digest) makes the file stale
    monkeypatch.setattr(autotuner, "library_digest", lambda jit: "another-build")
    tuned3, calls3, configs3, _ = _tuner(monkeypatch, tmp_path, [1.0, 3.0, 3.0])
    tuned3[(1,)](x, x, x, 8)
    assert len(calls3) > 1 and tuned3.config_for(x, x, x, 8) is configs3[0]


def test_autotuner_drops_candidates_that_are_out_of_reach_and_restores_arguments(monkeypatch, tmp_path):
    import torch

    tuned, calls, configs, _ = _tuner(monkeypatch, tmp_path, [1.0, 5.0, 1.02, 0.97])
    tuned.restore_value, tuned.reset_to_zero = ["x_ptr"], ["out_ptr"]
    x, out = torch.arange(8, dtype=torch.float32), torch.ones(8)
    seen_x = []
    hooked = configs[3]
    hooked.pre_hook = lambda args: seen_x.append(args["x_ptr"].clone())
    monkeypatch.setattr(tuned.jit, "run", lambda *a, grid, **kw: (calls.append(kw.get("variant")), a[0].add_(1), a[2].add_(1)))
    tuned[(1,)](x, x, out, 8)
    # variant 1 is five times slower: it is timed in the first pass only; the close ones race to the end
    assert calls.count(1) < calls.count(0) and calls.count(2) == calls.count(0)
    assert tuned.config_for(x, x, out, 8) is hooked  # 0.97 beats 1.0 by more than the 1% tolerance
    assert all(torch.equal(v, torch.arange(8, dtype=torch.float32)) for v in seen_x)  # restored before every launch
    assert set(tuned.timings[next(iter(tuned.timings))]) == {str(c) for c in configs}


def test_autotuner_skips_failing_configs(monkeypatch, tmp_path):
    tuned, calls, configs, _ = _tuner(monkeypatch, tmp_path, [1.0, 0.5])
    real_run = tuned.fn.run

    def run(*a, grid, **kw):
        if kw.get("variant") == 1:
            raise enceladus.CudaError("variant 1 cannot launch")
        real_run(*a, grid=grid, **kw)

    monkeypatch.setattr(tuned.fn, "run", run)
    x = np.zeros(8, np.float32)
    with pytest.warns(UserWarning, match="skipping"):
        tuned[(1,)](x, x, x, 8)
    assert tuned.config_for(x, x, x, 8) is configs[0]


def test_autotune_argument_validation():
    from enceladus_b200 import ops

    with pytest.raises(ValueError, match="at least one Config"):
        enceladus.autotune(configs=[], key=[])(ops.add_kernel)
    with pytest.raises(ValueError, match="unknown argument"):
        enceladus.autotune(configs=[enceladus.Config({})], key=["nope"])(ops.add_kernel)


def test_heuristics_compute_constexprs(monkeypatch):
    from enceladus_b200 import ops

    seen = {}
    monkeypatch.setattr(ops.add_kernel, "run", lambda *a, grid, **kw: seen.update(kw))
    h = enceladus.heuristics({"BLOCK": lambda args: enceladus.next_power_of_2(args["n"])})(ops.add_kernel)
    x = np.zeros(5, np.float32)
    h[(1,)](x, x, x, 5)
    assert seen["BLOCK"] == 8


def test_shard_range_partitions_exactly():
    for n, world, align in ((10, 3, 1), (4096, 8, 128), (1000, 8, 128), (5, 8, 1), (0, 2, 4)):
        spans = [edist.shard_range(n, r, world, align) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(s[0] % align == 0 for s in spans if s[0] < n)
    with pytest.raises(ValueError):
        edist.shard_range(4, 2, 2)


def test_exclusive_offsets_wrap_like_the_scan():
    t = np.array([2_000_000_000, 2_000_000_000, 5], np.int32)
    ex = edist.exclusive_offsets(t)
    assert ex.dtype == np.int32
    assert ex.tolist() == [0, 2_000_000_000, np.int64(4_000_000_000 - 2**32)]
    f = edist.exclusive_offsets(np.array([0.1, 0.2, 0.3], np.float32))
    assert f.dtype == np.float32 and f[0] == 0 and f[2] == np.float32(np.float32(0.1) + np.float32(0.2))


GLOO_WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np, torch, torch.distributed as dist
    sys.path.insert(0, {root!r})
    from enceladus_b200 import dist as edist
    from oracle import enceladus_oracle as O
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n = 100_003
    full = np.random.default_rng(0).integers(0, 1 << 30, n).astype(np.int32)   # wraps several times
    lo, hi = edist.shard_range(n, rank, world, 4)
    shard = torch.from_numpy(full[lo:hi].copy())
    total = lambda x: torch.from_numpy(np.array([x.numpy().astype(np.uint32).sum(dtype=np.uint32)]).view(np.int32))
    scan = lambda x, seed: torch.from_numpy((np.cumsum(x.numpy().astype(np.uint32), dtype=np.uint32)
                                             + seed.numpy().astype(np.uint32)).view(np.int32))
    got = edist.sharded_cumsum(shard, total, scan).numpy()
    want = O.cumsum(full)[lo:hi]
    assert np.array_equal(got, want), "cumsum shard mismatch on rank %d" % rank
    xs = np.random.default_rng(1).integers(0, 256, n).astype(np.int32)
    local = lambda x, bins, a, b: torch.from_numpy(O.histogram(x.numpy(), bins, a, b))
    h = edist.sharded_histogram(torch.from_numpy(xs[lo:hi].copy()), 256, 0.0, 256.0, local).numpy()
    assert np.array_equal(h, O.histogram(xs, 256, 0.0, 256.0)), "histogram mismatch on rank %d" % rank
    dist.barrier()
    dist.destroy_process_group()
    print("rank", rank, "ok")
""")


def test_two_rank_sharded_cumsum_and_histogram_over_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(GLOO_WORKER.format(root=str(ROOT)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29613", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{out}"
        assert f"rank {r} ok" in out


def test_warmup_and_explain_describe_the_native_kernel_without_launching(capsys):
    """`kernel.warmup()` / `kernel.explain()` (reference: src/enceladus/runtime/jit.py:527-573) resolve the
    native entry point and list the tile variants; neither needs a device."""
    from enceladus_b200 import _native as N
    from enceladus_b200 import ops

    x = np.zeros((4, 8), np.float32)
    ck = ops.softmax_kernel.warmup(x, x, 8, 8, 8, BLOCK=8)
    assert ck.entry == "enc_softmax" and ck.variant == -1 and len(ck.variants) == N.num_variants(N.K_SOFTMAX)
    q = np.zeros((1, 1, 128, 128), np.float16)
    text = ops.attention_kernel.explain(q, q, q, q, 1.0, 128, 128 * 128, 128, HEAD_DIM=128, BLOCK_M=128, BLOCK_N=128,
                                        CAUSAL=False, grid=(1, 1), variant=1)
    assert text == capsys.readouterr().out.rstrip("\n")
    assert "enc_attention_fwd" in text and "* variant 1" in text and "grid (1, 1, 1)" in text and "float16 (1, 1, 128, 128)" in text
    with pytest.raises(ValueError, match="variant 99"):
        ops.softmax_kernel.warmup(x, x, 8, 8, 8, BLOCK=8, variant=99)
    with pytest.raises(TypeError):
        ops.softmax_kernel.warmup(x, x, 8)


def test_piecewise_staging_plan_covers_every_unit_once_on_aligned_boundaries(monkeypatch):
    """Host logic of the piecewise NumPy staging (no device needed): pieces tile the units exactly, start on
    256-byte boundaries in every partitioned array, and arrays that cannot be cut fall back to one piece."""
    from enceladus_b200 import ops
    from enceladus_b200.runtime import jit

    monkeypatch.setattr(jit, "PIPELINE_MIN_BYTES", 1)
    monkeypatch.setattr(jit, "PIPELINE_PIECE_BYTES", 64 << 10)
    ad = ops.layernorm_kernel.adapter()
    m, n = 777, 1024
    x = np.zeros((m, n), np.float16)
    y, mean, rstd = np.empty_like(x), np.empty(m, np.float32), np.empty(m, np.float32)
    w = np.zeros(n, np.float16)
    bound = dict(x_ptr=x, y_ptr=y, w_ptr=w, b_ptr=w, mean_ptr=mean, rstd_ptr=rstd, stride_x=n, stride_y=n, n_cols=n, eps=1e-5, BLOCK=1024)
    hosts = ["x_ptr", "y_ptr", "w_ptr", "b_ptr", "mean_ptr", "rstd_ptr"]
    sp, pieces = jit._pipeline_plan(ad, bound, (m, 1, 1), hosts)
    assert sum(c for _, c in pieces) == m and [u for u, _ in pieces] == sorted({u for u, _ in pieces}) and len(pieces) >= 2
    assert all(u0 == pieces[i - 1][0] + pieces[i - 1][1] for i, (u0, _) in enumerate(pieces) if i)
    for name, per in sp.arrays.items():
        assert all((u0 * per * bound[name].itemsize) % 256 == 0 for u0, _ in pieces), name
    assert set(sp.arrays) == {"x_ptr", "y_ptr", "mean_ptr", "rstd_ptr"}  # w and b are shared, staged once
    # strided rows: the flat view would be a copy -> one piece
    bound2 = dict(bound, x_ptr=np.zeros((m, 2 * n), np.float16)[:, :n], stride_x=2 * n)
    assert jit._pipeline_plan(ad, bound2, (m, 1, 1), hosts) is None
    # too little data -> one piece
    monkeypatch.setattr(jit, "PIPELINE_MIN_BYTES", 1 << 30)
    assert jit._pipeline_plan(ad, bound, (m, 1, 1), hosts) is None
    # kernels without independent pieces have no split at all
    assert ops.histogram_kernel.adapter().split is None
    # the flat forward scan of a 32-bit type is cut along its row, each piece seeded by the one before
    monkeypatch.setattr(jit, "PIPELINE_MIN_BYTES", 1)
    cad = ops.cumsum_kernel.adapter()
    v = np.zeros(100003, np.int32)
    cb = dict(out_ptr=np.empty_like(v), in_ptr=v, n_rows=1, n_cols=v.size, stride_in=v.size, stride_out=v.size, REVERSE=False, BLOCK_M=1, BLOCK_N=131072)
    csp, cpieces = jit._pipeline_plan(cad, cb, (1, 1, 1), ["out_ptr", "in_ptr"])
    assert csp.chain is not None and sum(c for _, c in cpieces) == v.size and all(type(c) is int and (u * 4) % 256 == 0 for u, c in cpieces)
    re = csp.rebind(cpieces[0][1])
    assert re["n_cols"] == cpieces[0][1] and re["BLOCK_N"] >= re["n_cols"] and csp.grid(cpieces[0][1]) == (1, 1, 1)
    assert jit._pipeline_plan(cad, dict(cb, REVERSE=True), (1, 1, 1), ["out_ptr", "in_ptr"]) is None
    h16 = np.zeros(100003, np.float16)
    assert jit._pipeline_plan(cad, dict(cb, in_ptr=h16, out_ptr=np.empty_like(h16)), (1, 1, 1), ["out_ptr", "in_ptr"]) is None


def test_same_name_kernel_with_another_body_is_refused():
    """The body of a `@jit` kernel is never executed: a definition whose code is not the reference's kernel of
    that name must not be served by the built-in kernel."""
    @enceladus.jit
    def add_kernel(x_ptr, y_ptr, out_ptr, n, BLOCK: tl.constexpr):
        offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
        mask = offs < n
        tl.store(out_ptr + offs, tl.load(x_ptr + offs, mask=mask) - tl.load(y_ptr + offs, mask=mask), mask=mask)

    x = np.zeros(8, np.float32)
    with pytest.raises(NotImplementedError, match="not the reference's kernel of that name"):
        add_kernel[(1,)](x, x, x, 8, BLOCK=8)

    # the reference's own body (examples/01_vector_add.py:15-22) is accepted, however it is formatted
    @enceladus.jit
    def add_kernel(x_ptr, y_ptr, out_ptr, n, BLOCK: tl.constexpr):  # noqa: F811
        offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
        mask = offs < n  # a comment does not change the fingerprint

        tl.store(out_ptr + offs, tl.load(x_ptr + offs, mask=mask) + tl.load(y_ptr + offs, mask=mask), mask=mask)

    assert add_kernel.adapter().name == "add_kernel"

    @enceladus.jit
    def add_kernel(x_ptr, y_ptr, out_ptr, n, BLOCK: tl.constexpr):  # noqa: F811
        """Documentation only."""
        ...

    assert add_kernel.adapter().name == "add_kernel"
    from enceladus_b200 import ops

    for name in registry.kernels():  # every kernel the package itself defines resolves
        k = getattr(ops, name, None)
        if k is not None and hasattr(k, "adapter"):
            assert k.adapter().name == name


def test_tensors_on_two_devices_are_refused(monkeypatch):
    """All array arguments of a launch must live on one device; checked before anything reaches the library."""
    from enceladus_b200.runtime import interop, jit

    class FakeDevice:
        def __init__(self, index):
            self.index = index

        def __eq__(self, other):
            return self.index == other.index

        def __ne__(self, other):
            return self.index != other.index

        def __repr__(self):
            return f"cuda:{self.index}"

    class FakeTensor:
        is_cuda = True

        def __init__(self, index):
            self.device = FakeDevice(index)

    monkeypatch.setattr(interop, "tensor_type", lambda: FakeTensor)
    from enceladus_b200 import ops

    ad = ops.add_kernel.adapter()
    bound = {"x_ptr": FakeTensor(0), "y_ptr": FakeTensor(0), "out_ptr": FakeTensor(1), "n": 4, "BLOCK": 4}
    with pytest.raises(ValueError, match=r"`out_ptr` lives on cuda:1 but `x_ptr` lives on cuda:0"):
        jit.launch(ad, bound, (1, 1, 1), -1, None)
