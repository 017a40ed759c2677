"""Seeded synthetic inputs for the benchmark configurations.

No public dataset is involved: these shapes and value distributions *are* the workload.  Every
generator takes a seed and returns host NumPy arrays, so the CUDA path and the CPU checker are fed the
identical bytes.
"""

from __future__ import annotations

import numpy as np


def zipf_clipped(rng: np.random.Generator, n: int, s: float, nbins: int) -> np.ndarray:
    """Zipf(s) samples clipped to `nbins - 1`, as int32, by inverse CDF on the truncated support.

    P(k) ~ k^-s for k = 1, 2, ...; every k >= nbins-1 is lumped into the last bin, which is the
    distribution `np.minimum(rng.zipf(s, n), nbins - 1)` has, at a fraction of the sampling cost.
    """
    from scipy.special import zeta

    k = np.arange(1, nbins - 1, dtype=np.float64)
    cdf = np.concatenate([[0.0], np.cumsum(k ** (-s) / zeta(s, 1))])  # cdf[j] = P(K <= j)
    out = np.empty(n, np.int32)
    step = 1 << 24
    for i in range(0, n, step):
        u = rng.random(min(step, n - i))
        out[i : i + step] = np.minimum(np.searchsorted(cdf, u, side="right"), nbins - 1)
    return out
