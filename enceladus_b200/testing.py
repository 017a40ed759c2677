"""Benchmarking and comparison helpers (counterpart of src/enceladus/testing.py)."""

from __future__ import annotations

import statistics
from collections.abc import Callable
from typing import Any

import numpy as np


def do_bench(fn: Callable[[], Any], warmup_ms: float = 50.0, rep: int = 20, return_mode: str = "median",
             flush_l2: bool = False) -> float | list[float]:
    """Times `fn` on the GPU with CUDA events on the current stream and returns milliseconds.

    `fn` must launch its work on torch's current CUDA stream with device-resident arguments; a launch
    that synchronises internally (for example one with NumPy arguments) measures its copies too.

    Args:
        fn: A function that launches one or more kernels.
        warmup_ms: GPU time to spend warming up before measuring (at least 3 runs).
        rep: The number of timed repetitions, each bracketed by its own pair of events.
        return_mode: "median", "min", "mean", or "all" (a list of every sample).
        flush_l2: Overwrite a buffer larger than L2 before each repetition.
    """
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("do_bench needs a CUDA device")
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush_l2 else None
    torch.cuda.synchronize()
    spent, runs = 0.0, 0
    while spent < warmup_ms or runs < 3:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        t = a.elapsed_time(b)
        if t <= 0.0:
            raise RuntimeError("do_bench measured no GPU work; fn must launch kernels on the current stream")
        spent += t
        runs += 1
        if runs > 10000:
            break
    samples = []
    for _ in range(rep):
        if scratch is not None:
            scratch.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        samples.append(a.elapsed_time(b))
    if return_mode == "all":
        return samples
    if return_mode == "min":
        return min(samples)
    if return_mode == "mean":
        return statistics.fmean(samples)
    return statistics.median(samples)


def default_tolerance(dtype: Any) -> tuple[float, float]:
    """Returns (atol, rtol) suited to comparing results of `dtype`."""
    name = str(np.dtype(dtype.to_numpy() if hasattr(dtype, "to_numpy") else dtype))
    if name == "bfloat16":
        return 2e-2, 2e-2
    if name == "float16":
        return 2e-3, 2e-3
    if name == "float32":
        return 1e-5, 1e-5
    return 0.0, 0.0


def _host(x: Any) -> np.ndarray:
    if hasattr(x, "detach"):  # torch tensor
        import torch

        x = x.detach().cpu()
        if x.dtype == torch.bfloat16:
            import ml_dtypes

            return x.view(torch.int16).numpy().view(ml_dtypes.bfloat16)
        return x.numpy()
    return np.asarray(x)


def assert_close(actual: Any, expected: Any, atol: float | None = None, rtol: float | None = None):
    """Asserts that two arrays match within dtype-aware tolerances; integers must be equal."""
    a, e = _host(actual), _host(expected)
    d_atol, d_rtol = default_tolerance(a.dtype)
    wide = lambda v: v.astype(np.float32) if v.dtype.kind == "V" or (v.dtype.kind == "f" and v.dtype.itemsize == 2) else v  # noqa: E731
    np.testing.assert_allclose(wide(a), wide(e), atol=d_atol if atol is None else atol,
                               rtol=d_rtol if rtol is None else rtol)
