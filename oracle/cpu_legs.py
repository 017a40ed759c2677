"""Timed CPU legs of the benchmark: the reference's own CPU path on this host's cores.

TEST AND MEASUREMENT INFRASTRUCTURE ONLY (used by `bench.py`'s `cpu_baseline` legs and `--impl reference`).

For every workload of the kernel set there is a leg that runs a bounded SAMPLE of the workload through
  (i)  the reference interpreter (`ENCELADUS_INTERPRET=1`, the example's own host wrapper: kind "reference"), and
  (ii) the example's float64 NumPy `reference()` (reported beside it as `numpy_reference`).
When `oracle/_ref/` is not installed the NumPy restatement in `enceladus_oracle.py` stands in (kind "port").

The interpreter is single-threaded Python (one program instance after the other, interp.py:801-825), so a leg
whose sample cuts into independent pieces (rows, elements, heads: everything except the matmuls, whose time is
BLAS inside `tl.dot`) is run by a pool of forked worker processes, one per host core, each on its slice of the
sample: that is "all the host threads it can use".  The pool is forked before CUDA is initialised.  Timing is
wall clock around the pool's map; the value is units of the sample / that time, in the workload's own unit.

Tile sizes are free parameters of an interpreted launch (they change float results in the last ulp only) and
are stated in every `sample` string.
"""

from __future__ import annotations

import math
import multiprocessing as mp
import os
import time

import ml_dtypes
import numpy as np

BF16 = np.dtype(ml_dtypes.bfloat16)

SAMPLE_BYTES_MAX = 64 << 20  # input bytes of a sample, at most
_STATE: dict = {}  # leg, inputs, ref: set in the parent before the pool is forked, read by the workers


def cores() -> int:
    return len(os.sched_getaffinity(0))


def blas_threads() -> int:
    try:
        import threadpoolctl

        return max((d.get("num_threads", 1) for d in threadpoolctl.threadpool_info() if d.get("user_api") == "blas"), default=1)
    except Exception:  # noqa: BLE001
        return 1


def _f16(x: np.ndarray) -> np.ndarray:
    """float32 -> float16, round to nearest even; torch's vectorised conversion when it is there (NumPy converts
    one element at a time, which for a 8192 x 8192 operand takes longer than the leg it feeds)."""
    try:
        import torch

        return torch.from_numpy(np.ascontiguousarray(x)).half().numpy()
    except Exception:  # noqa: BLE001
        return x.astype(np.float16)


def _bf16(rng, shape, scale=1.0, shift=0.0):
    return (shift + scale * rng.standard_normal(shape)).astype(np.float32).astype(BF16)


# ---- the legs ------------------------------------------------------------------------------------------
# make(units_hint) -> inputs dict with "n" = number of splittable pieces along axis 0 of the marked arrays
# interp(ref, inputs, lo, hi) / numpy_ref(ref, inputs, lo, hi) / port(inputs, lo, hi) run pieces [lo, hi)
# units(inputs, lo, hi) -> algorithmic bytes or flops of those pieces
class Leg:
    unit = "GB/s"
    parallel = True        # pieces are independent: fork one worker per core
    tiles = ""             # interpreter tile sizes, for the sample string
    piece = "rows"
    per_piece_probe = 8    # pieces in the timing probe

    def make(self, pieces: int) -> dict: ...
    def interp(self, ref, d, lo, hi): ...
    def numpy_ref(self, ref, d, lo, hi): ...
    def port(self, d, lo, hi): ...
    def units(self, d, lo, hi) -> float: ...

    def numpy_units(self, d, lo, hi) -> float:  # units the NumPy path processes for pieces [lo, hi)
        return self.units(d, lo, hi)

    numpy_note = ""
    full_pieces = 0        # pieces of the whole workload
    piece_bytes = 0        # input bytes of one piece (caps the sample: generating and holding it is not what is timed)


class Softmax(Leg):
    def __init__(self, cols):
        self.cols, self.full_pieces, self.tiles, self.piece_bytes = cols, 4096, f"BLOCK={cols}", cols * 4

    def make(self, pieces):
        return {"x": np.random.default_rng(0).standard_normal((pieces, self.cols)).astype(np.float32) * 4}

    def interp(self, ref, d, lo, hi):
        return ref.example("02_softmax").softmax(d["x"][lo:hi])

    def numpy_ref(self, ref, d, lo, hi):
        return ref.example("02_softmax").reference(d["x"][lo:hi])

    def port(self, d, lo, hi):
        from oracle import enceladus_oracle as O

        return O.softmax(d["x"][lo:hi])

    def units(self, d, lo, hi):
        return 2.0 * (hi - lo) * self.cols * 4


class Norm(Leg):
    def __init__(self, kind):
        self.kind, self.full_pieces, self.piece_bytes = kind, 16384, 4096 * 2
        self.tiles = "BLOCK=1024" if kind == "layernorm" else "BLOCK=4096"

    def make(self, pieces):
        r = np.random.default_rng(0)
        return {"x": _bf16(r, (pieces, 4096)), "w": _bf16(r, 4096, 0.1, 1.0), "b": _bf16(r, 4096, 0.1)}

    def interp(self, ref, d, lo, hi):
        if self.kind == "layernorm":
            return ref.example("03_layernorm").layernorm(d["x"][lo:hi], d["w"], d["b"], 1e-5)
        return ref.example("06_rmsnorm").rmsnorm(d["x"][lo:hi], d["w"], 1e-6)

    def numpy_ref(self, ref, d, lo, hi):
        if self.kind == "layernorm":
            return ref.example("03_layernorm").reference(d["x"][lo:hi], d["w"], d["b"], 1e-5)
        return ref.example("06_rmsnorm").reference(d["x"][lo:hi], d["w"], 1e-6)

    def port(self, d, lo, hi):
        from oracle import enceladus_oracle as O

        return O.layernorm(d["x"][lo:hi], d["w"], d["b"], 1e-5) if self.kind == "layernorm" else O.rmsnorm(d["x"][lo:hi], d["w"], 1e-6)

    def units(self, d, lo, hi):
        return 2.0 * (hi - lo) * 4096 * 2


class TanhGelu(Leg):
    """The benchmark's tanh-GELU is not one of the reference's examples; it is the DSL kernel below, written
    against the reference's own `enceladus.language` and executed by its interpreter (the kernel that also
    produced tests/golden/gelu.npz).  The NumPy path is the same formula in float64."""

    BLOCK = 65536
    piece = "blocks of 65536 elements"

    def __init__(self):
        self.full_pieces, self.tiles, self._kernel, self.piece_bytes = (1 << 28) // self.BLOCK, f"BLOCK={self.BLOCK}", None, self.BLOCK * 4

    def make(self, pieces):
        return {"x": (np.random.default_rng(0).standard_normal(pieces * self.BLOCK) * 2).astype(np.float32).reshape(pieces, self.BLOCK)}

    def kernel(self, ref):
        if self._kernel is None:
            enceladus = ref.package
            import enceladus.language as tl

            @enceladus.jit
            def tanh_gelu_kernel(x_ptr, out_ptr, n, BLOCK: tl.constexpr):
                offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
                mask = offs < n
                x = tl.load(x_ptr + offs, mask=mask).to(tl.float32)
                inner = 0.7978845608028654 * (x + 0.044715 * x * x * x)
                tl.store(out_ptr + offs, 0.5 * x * (1.0 + tl.tanh(inner)), mask=mask)

            self._kernel = tanh_gelu_kernel
        return self._kernel

    def interp(self, ref, d, lo, hi):
        x = d["x"][lo:hi].reshape(-1)
        y = np.empty_like(x)
        from oracle.ref_runtime import interpreting

        with interpreting():
            self.kernel(ref)[(hi - lo,)](x, y, x.size, BLOCK=self.BLOCK)
        return y

    def numpy_ref(self, ref, d, lo, hi):
        x = d["x"][lo:hi].astype(np.float64)
        return (0.5 * x * (1 + np.tanh(0.7978845608028654 * (x + 0.044715 * x**3)))).astype(np.float32)

    def port(self, d, lo, hi):
        from oracle import enceladus_oracle as O

        return O.gelu_tanh(d["x"][lo:hi].reshape(-1))

    def units(self, d, lo, hi):
        return 2.0 * (hi - lo) * self.BLOCK * 4


class FusedMatmul(Leg):
    unit, parallel, piece, per_piece_probe = "TFLOP/s", False, "blocks of 256 rows of A", 1

    def __init__(self, m, n, k):
        self.m, self.n, self.k, self.full_pieces = m, n, k, m // 256
        self.tiles = "BM=256 BN=512 BK=512, BLAS threads = %d" % blas_threads()

    def make(self, pieces):
        r = np.random.default_rng(0)
        sc = np.float32(1 / math.sqrt(self.k))
        return {"a": _f16((r.random((pieces * 256, self.k), dtype=np.float32) * 2 - 1) * sc),
                "b": _f16((r.random((self.k, self.n), dtype=np.float32) * 2 - 1) * sc),
                "bias": (0.1 * r.standard_normal(self.n, dtype=np.float32)).astype(np.float16)}

    def interp(self, ref, d, lo, hi):
        return ref.example("07_matmul_fused").matmul_bias_gelu(d["a"][lo * 256 : hi * 256], d["b"], d["bias"], bm=256, bn=512, bk=512)

    # The example's reference() converts both float16 operands to float64 (about 0.2 microseconds per element of B
    # in NumPy) and applies np.vectorize(math.erf): the NumPy path takes the first 32 rows of each 256-row block
    # against the first 1024 columns of B.
    numpy_note = " (first 32 rows of each block x first 1024 columns of B)"

    def numpy_ref(self, ref, d, lo, hi):
        rows = np.concatenate([np.arange(p * 256, p * 256 + 32) for p in range(lo, hi)])
        return ref.example("07_matmul_fused").reference(d["a"][rows], d["b"][:, :1024], d["bias"][:1024])

    def numpy_units(self, d, lo, hi):
        return 2.0 * (hi - lo) * 32 * 1024 * self.k

    def port(self, d, lo, hi):
        from oracle import enceladus_oracle as O

        return O.matmul_bias_gelu(d["a"][lo * 256 : hi * 256], d["b"], d["bias"], 512)

    def units(self, d, lo, hi):
        return 2.0 * (hi - lo) * 256 * self.n * self.k


class Attention(Leg):
    unit, piece, per_piece_probe = "TFLOP/s", "(batch, head) slices", 1
    tiles = "BLOCK_M=128 BLOCK_N=128"

    def __init__(self, causal):
        self.causal, self.full_pieces = causal, 256

    def make(self, pieces):
        r = np.random.default_rng(0)
        return {k: _bf16(r, (pieces, 1, 4096, 128)) for k in "qkv"}

    def interp(self, ref, d, lo, hi):
        return ref.example("08_flash_attention").attention(d["q"][lo:hi], d["k"][lo:hi], d["v"][lo:hi], self.causal)

    def numpy_ref(self, ref, d, lo, hi):
        return ref.example("08_flash_attention").reference(d["q"][lo:hi], d["k"][lo:hi], d["v"][lo:hi], self.causal)

    def port(self, d, lo, hi):
        from oracle import enceladus_oracle as O

        return O.attention(d["q"][lo:hi], d["k"][lo:hi], d["v"][lo:hi], self.causal, None, 128, 128)

    def units(self, d, lo, hi):
        return 4.0 * (hi - lo) * 4096 * 4096 * 128 / (2 if self.causal else 1)


class Histogram(Leg):
    """Through the interpreter a colliding `tl.atomic_add` is applied one element at a time in Python
    (src/enceladus/language/ops.py:1893-1901), about 2 microseconds per element, so its sample is small; the
    example's `reference()` (float32 bin arithmetic + np.bincount) takes a larger one."""

    BLOCK = 1 << 14
    piece = "blocks of 16384 elements"

    def __init__(self, kind):
        self.kind, self.bins, self.full_pieces = kind, 256 if kind == "uniform256" else 4096, (1 << 30) // self.BLOCK
        self.piece_bytes = self.BLOCK * 4
        self.tiles = "BLOCK=1024"

    def make(self, pieces):
        n = pieces * self.BLOCK
        if self.kind == "uniform256":
            x = np.random.default_rng(0).integers(0, 256, n).astype(np.int32)
        else:
            from enceladus_b200.workloads import zipf_clipped

            x = zipf_clipped(np.random.default_rng(0), n, 1.1, 4096)
        return {"x": x.reshape(pieces, self.BLOCK)}

    def interp(self, ref, d, lo, hi):
        return ref.example("09_histogram").histogram(d["x"][lo:hi].reshape(-1), self.bins, 0.0, float(self.bins))

    def numpy_ref(self, ref, d, lo, hi):
        return ref.example("09_histogram").reference(d["x"][lo:hi].reshape(-1), self.bins, 0.0, float(self.bins))

    def port(self, d, lo, hi):
        from oracle import enceladus_oracle as O

        return O.histogram(d["x"][lo:hi].reshape(-1), self.bins, 0.0, float(self.bins))

    def units(self, d, lo, hi):
        return float(hi - lo) * self.BLOCK * 4


class Cumsum(Leg):
    """The flat 2^30 / 2^28 scan is longer than any tile the reference can express (one whole row per tile, at
    most 65536 elements: examples/10_cumsum.py:17-25), so the interpreter leg scans the sample as rows of 65536,
    which moves the same bytes through the same `tl.cumsum`; the NumPy path is the example's `reference()`."""

    ROW = 65536
    piece = "rows of 65536 elements"

    def __init__(self, kind):
        self.kind, self.full_pieces = kind, ((1 << 30) if kind == "i32" else (1 << 28)) // self.ROW
        self.piece_bytes = self.ROW * 4
        self.tiles = "BLOCK_M=1 BLOCK_N=65536"

    def make(self, pieces):
        r = np.random.default_rng(0)
        if self.kind == "i32":
            return {"x": r.integers(0, 16, (pieces, self.ROW)).astype(np.int32)}
        return {"x": r.standard_normal((pieces, self.ROW)).astype(np.float32)}

    def interp(self, ref, d, lo, hi):
        return ref.example("10_cumsum").cumsum(d["x"][lo:hi])

    def numpy_ref(self, ref, d, lo, hi):
        return ref.example("10_cumsum").reference(d["x"][lo:hi])

    def port(self, d, lo, hi):
        from oracle import enceladus_oracle as O

        return O.cumsum(d["x"][lo:hi])

    def units(self, d, lo, hi):
        return 2.0 * (hi - lo) * self.ROW * 4


LEGS = {
    "softmax_f32_4096x1024": lambda: Softmax(1024),
    "softmax_f32_4096x4096": lambda: Softmax(4096),
    "layernorm_bf16_16384x4096": lambda: Norm("layernorm"),
    "rmsnorm_bf16_16384x4096": lambda: Norm("rmsnorm"),
    "gelu_tanh_f32_2p28": TanhGelu,
    "matmul_bias_gelu_f16_8192x8192x8192": lambda: FusedMatmul(8192, 8192, 8192),
    "matmul_bias_gelu_f16_4096x4096x16384": lambda: FusedMatmul(4096, 4096, 16384),
    "attention_bf16_8x32x4096x128_full": lambda: Attention(False),
    "attention_bf16_8x32x4096x128_causal": lambda: Attention(True),
    "histogram_i32_2p30_uniform256": lambda: Histogram("uniform256"),
    "histogram_i32_2p30_zipf4096": lambda: Histogram("zipf4096"),
    "cumsum_i32_2p30": lambda: Cumsum("i32"),
    "cumsum_f32_2p28": lambda: Cumsum("f32"),
}


# ---- running a leg -----------------------------------------------------------------------------------
def _run(which: str, lo: int, hi: int):
    leg, d, ref = _STATE["leg"], _STATE["inputs"], _STATE["ref"]
    if which == "interp":
        return leg.interp(ref, d, lo, hi)
    if which == "numpy":
        return leg.numpy_ref(ref, d, lo, hi)
    return leg.port(d, lo, hi)


def _worker(task):
    which, lo, hi = task
    if hi > lo:
        _run(which, lo, hi)
    return hi - lo


def _limit_blas_in_worker():
    try:  # one BLAS thread per worker: the workers are the parallelism
        import threadpoolctl

        threadpoolctl.threadpool_limits(1)
    except Exception:  # noqa: BLE001
        pass


class Runner:
    """A leg with its sample in memory and (for parallel legs) a forked pool.  `step(which)` runs the whole sample
    once and returns (seconds, units)."""

    def __init__(self, name: str, budget_s: float, workers: int | None = None, use_ref: bool = True) -> None:
        from oracle import ref_runtime

        self.name = name
        self.leg = LEGS[name]()
        self.ref = ref_runtime.load() if use_ref else None
        self.kind = "reference" if self.ref is not None else "port"
        self.which = "interp" if self.ref is not None else "port"
        self.workers = (workers or cores()) if self.leg.parallel else 1
        # probe: seconds per piece in one process
        probe_n = self.leg.per_piece_probe
        _STATE.update(leg=self.leg, inputs=self.leg.make(probe_n), ref=self.ref)
        t0 = time.perf_counter()
        _run(self.which, 0, probe_n)
        dt = time.perf_counter() - t0
        if dt < 0.5:  # short enough for imports and first-call costs to matter: time a second, warm run
            t0 = time.perf_counter()
            _run(self.which, 0, probe_n)
            dt = time.perf_counter() - t0
        per_piece = max(dt / probe_n, 1e-6)
        pieces = int(budget_s * self.workers / per_piece)
        if self.leg.piece_bytes:
            pieces = min(pieces, max(self.workers, SAMPLE_BYTES_MAX // self.leg.piece_bytes))
        pieces = max(self.workers, min(self.leg.full_pieces, pieces))
        if self.leg.parallel:
            pieces -= pieces % self.workers
        self.pieces = max(pieces, 1)
        self.inputs = _STATE["inputs"] if self.pieces == probe_n else self.leg.make(self.pieces)
        _STATE.update(inputs=self.inputs)
        self.pool = None
        if self.leg.parallel and self.workers > 1:
            self.pool = mp.get_context("fork").Pool(self.workers, initializer=_limit_blas_in_worker)
            self.pool.map(_worker, [(self.which, 0, 0)] * self.workers)  # workers are up before any timing

    def tasks(self, which: str, pieces: int):
        per = -(-pieces // self.workers)
        return [(which, i * per, min(pieces, (i + 1) * per)) for i in range(self.workers)]

    def step(self, which: str | None = None, pieces: int | None = None) -> tuple[float, float]:
        which, pieces = which or self.which, pieces or self.pieces
        t0 = time.perf_counter()
        if self.pool is not None:
            self.pool.map(_worker, self.tasks(which, pieces), chunksize=1)
        else:
            _run(which, 0, pieces)
        return time.perf_counter() - t0, self.leg.units(self.inputs, 0, pieces)

    def close(self) -> None:
        if self.pool is not None:
            self.pool.close()
            self.pool.join()
            self.pool = None
        _STATE.clear()

    def sample(self, pieces: int | None = None) -> str:
        p = pieces or self.pieces
        how = (f"{self.workers} forked worker processes, one slice each" if self.pool is not None
               else f"one process, BLAS threads = {blas_threads()}")
        what = ("reference interpreter (ENCELADUS_INTERPRET=1) via the example's host wrapper" if self.kind == "reference"
                else "NumPy restatement of the reference interpreter (oracle/_ref not installed)")
        return (f"{p} of {self.leg.full_pieces} {self.leg.piece}; {what}; tiles {self.leg.tiles}; {how}; "
                f"host cores = {cores()}, numpy {np.__version__}, ml_dtypes {ml_dtypes.__version__}")


def baseline(name: str, budget_s: float = 3.0, numpy_budget_s: float = 1.0) -> dict | None:
    """`cpu_baseline` object of one workload: the interpreter on all cores, plus the example's NumPy reference()."""
    if name not in LEGS:
        return None
    scale = 1e9
    r = Runner(name, budget_s)
    try:
        scale = 1e9 if r.leg.unit == "GB/s" else 1e12
        dt, units = r.step()
        out = {"value": units / dt / scale, "unit": r.leg.unit, "cores": r.workers if r.leg.parallel else blas_threads(),
               "kind": r.kind, "sample": r.sample() + f"; {dt:.2f} s"}
        if r.ref is not None:
            # the float64 NumPy path on (at most) the same sample, sized by a one-piece probe
            t0 = time.perf_counter()
            _run("numpy", 0, 1)
            per = max(time.perf_counter() - t0, 1e-6)
            if per >= numpy_budget_s:  # one piece already fills the budget: that run is the measurement
                pieces, dt2, units2, how = 1, per, r.leg.numpy_units(r.inputs, 0, 1), "one process"
            else:
                pieces = max(1, min(r.pieces, int(numpy_budget_s * r.workers / per)))
                if r.pool is not None:
                    pieces = max(r.workers, pieces - pieces % r.workers)
                dt2, _ = r.step("numpy", pieces)
                units2 = r.leg.numpy_units(r.inputs, 0, pieces)
                how = f"{r.workers} worker processes" if r.pool is not None else "one process"
            out["numpy_reference"] = {"value": units2 / dt2 / scale, "unit": r.leg.unit,
                                      "sample": f"{pieces} {r.leg.piece}{r.leg.numpy_note} through the example's float64 reference(), {how}; {dt2:.2f} s"}
        return out
    finally:
        r.close()
