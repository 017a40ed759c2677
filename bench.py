"""Benchmark of the kernel set on B200: per-kernel HBM GB/s or TFLOP/s against the measured roofline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--kernels all|none|a,b,...]
                    [--impl ours|reference] [--scaling weak|strong] [--no-e2e] [--no-cpu-baseline]

Prints ONE JSON line.  The headline workload (default `layernorm`: LayerNorm over bf16 [16384, 4096]) is
timed for exactly K steps after W warm-up steps; `roofline.per_kernel` carries one entry for every workload
of the kernel set, each timed the same way with its own step count.  A step is one launch of the kernel over
one batch of seeded synthetic input that is already resident in HBM.  Between steps the kernels rotate
through several buffer sets whose total size exceeds L2 several times, so every step reads from DRAM.

  value          algorithmic bytes (or FLOPs) of all ranks / device time (CUDA events, max over ranks)
  e2e            the same metric through the public launch path with HOST (pinned NumPy) arguments:
                 host->device copy, kernel, device->host copy inside the timed region; `e2e.pcie` holds the
                 pinned copy bandwidths measured in the same run and `e2e.frac` = the time the copies alone
                 need at those bandwidths / the measured time
  roofline       achieved / measured peak (MEASURED_PEAKS.json if present, else the stated fallback)
  cpu_baseline   the reference's own CPU path (its interpreter, ENCELADUS_INTERPRET=1, installed under
                 oracle/_ref by oracle/build_ref.py) on this host's cores, bounded sample, with the example's
                 float64 NumPy reference() beside it; N = 1 only, measured before CUDA is initialised
  verified       every row is checked in-run against an independent computation of the same result

N > 1 (under torchrun).  `--scaling weak` (default): every rank runs the same per-GPU workload; `--scaling
strong`: the configuration itself is cut into contiguous shards (rows, elements, M-blocks, (batch, head)
slices).  Either way the histogram adds its all-reduce of the bins and the flat cumsum its all-gather of shard
totals inside the timed region, and both results are verified across ranks.  `--impl reference` times the
reference's CPU path on all host cores (rank 0 only).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
L2_BYTES = 126 << 20
ROTATE_BYTES = 1 << 30  # total size of the rotating buffer sets for workloads smaller than this

# dram__bytes_read.sum + dram__bytes_write.sum per launch (bytes), from the `ncu --set full` captures
# summarised under profiles/ (one file per workload, with the capturing command).  The 2^30 / 2^28-element
# workloads were captured at 2^27 elements (few GB on the device under the profiler) and are scaled by
# the element count: their traffic is proportional to it.
NCU_TRAFFIC: dict[str, float | None] = {
    "layernorm_bf16_16384x4096": 219_303_936,       # profiles/layernorm.md
    "rmsnorm_bf16_16384x4096": 216_850_688,         # profiles/rmsnorm.md
    "softmax_f32_4096x1024": 16_802_304,            # profiles/softmax.md (the 16 MiB output stays in L2)
    "gelu_tanh_f32_2p28": 2_100_776_000,            # profiles/gelu.md
    "histogram_i32_2p30_uniform256": 8 * 540_655_616,   # profiles/hist_uniform256.md, captured at 2^27
    "histogram_i32_2p30_zipf4096": 8 * 540_067_328,     # profiles/hist_zipf4096.md, captured at 2^27
    "cumsum_i32_2p30": 8 * 1_015_634_688,           # profiles/cumsum_i32.md, captured at 2^27
    "cumsum_f32_2p28": 2 * 1_015_431_168,           # profiles/cumsum_f32.md, captured at 2^27
    "matmul_bias_gelu_f16_8192x8192x8192": 1_048_525_312,   # profiles/matmul.md
    "matmul_int8_8192x8192x8192": 571_891_712,              # profiles/matmul_int8.md
    "attention_bf16_8x32x4096x128_full": 1_056_008_704,     # profiles/attention_full.md
    "attention_bf16_8x32x4096x128_causal": 1_051_185_408,   # profiles/attention_causal.md
}

USE_GRAPH = True
RANK = int(os.environ.get("RANK", "0"))
LOCAL_RANK = int(os.environ.get("LOCAL_RANK", "0"))
WORLD = int(os.environ.get("WORLD_SIZE", "1"))


def peaks() -> tuple[dict, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            if d.get("hbm_gbs") and d.get("bf16_tflops"):
                return d, "measured"
        except ValueError:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ---------------------------------------------------------------------------------------------------
# Workloads.  Each entry builds a dict with: make(i) -> argument set number i on the device, run(set),
# verify(set) -> bool (after run(set)), work (algorithmic bytes or flops per launch on this rank), unit,
# bound, dtype, and optionally host()/run_host() for the end-to-end path.
# `shard` = (rank, world) cuts the configuration itself (strong scaling); None = the whole configuration.
# ---------------------------------------------------------------------------------------------------
def _bf16_host(shape, rng, scale=1.0, shift=0.0):
    import ml_dtypes

    return (shift + scale * rng.standard_normal(shape)).astype(np.float32).astype(ml_dtypes.bfloat16)


def _f16_host(x: np.ndarray) -> np.ndarray:
    import torch

    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).half().numpy()


def workloads(scale: float = 1.0, shard: tuple[int, int] | None = None):
    import torch

    from enceladus_b200 import _native as N
    from enceladus_b200 import dist as edist
    from enceladus_b200 import ops

    W = {}

    def gen(seed):
        g = torch.Generator(device="cuda")
        g.manual_seed(seed)
        return g

    def part(n, align=1):
        """This rank's share of n units under strong scaling, the whole n otherwise."""
        if shard is None:
            return n
        lo, hi = edist.shard_range(n, shard[0], shard[1], align)
        return hi - lo

    def close(got, want, atol, rtol):
        return bool(torch.isfinite(got.float()).all()) and bool(torch.allclose(got.float(), want.float(), atol=atol, rtol=rtol))

    # ---- config 1: softmax fp32 [4096, 1024] ----
    def softmax_wl(n=1024):
        m_full = 4096
        m = part(m_full)

        def verify(s):  # rows sum to one, and 64 rows against torch
            x, y = s
            rows = torch.linspace(0, m - 1, 64, device="cuda").long()
            return bool((y.sum(1, dtype=torch.float64) - 1).abs().max() < 1e-5) and close(y[rows], torch.softmax(x[rows], 1), 1e-6, 1e-5)

        return dict(
            name=f"softmax_f32_{m_full}x{n}", kernel="softmax", jit=ops.softmax_kernel, unit="GB/s", bound="hbm", dtype="f32",
            work=2 * m * n * 4, set_bytes=2 * m * n * 4,
            make=lambda i: (torch.randn(m, n, device="cuda", generator=gen(i)) * 4, torch.empty(m, n, device="cuda")),
            run=lambda s: ops.softmax_kernel[(m,)](s[1], s[0], n, n, n, BLOCK=n), verify=verify,
            host=lambda: (np.random.default_rng(0).standard_normal((m, n)).astype(np.float32) * 4,),
            run_host=lambda h: ops.softmax(h[0]))

    # ---- config 2: LayerNorm / RMSNorm bf16 [16384, 4096], tanh-GELU fp32 2^28 ----
    def norm_wl(kind):
        m_full, n = 16384, 4096
        m = part(m_full)

        def make(i):
            g = gen(i)
            x = torch.randn(m, n, device="cuda", generator=g).to(torch.bfloat16)
            w = (1 + 0.1 * torch.randn(n, device="cuda", generator=g)).to(torch.bfloat16)
            b = (0.1 * torch.randn(n, device="cuda", generator=g)).to(torch.bfloat16)
            y = torch.empty_like(x)
            return x, w, b, y, torch.empty(m, device="cuda"), torch.empty(m, device="cuda")

        def host():
            r = np.random.default_rng(0)
            return _bf16_host((m, n), r), _bf16_host(n, r, 0.1, 1.0), _bf16_host(n, r, 0.1)

        def verify(s):  # 256 rows against the float32 formula in torch (bf16 output tolerance), statistics at 1e-5
            x, w, b, y, mean, rstd = s
            rows = torch.linspace(0, m - 1, 256, device="cuda").long()
            xf = x[rows].float()
            if kind == "layernorm":
                mu = xf.mean(1, keepdim=True)
                var = ((xf - mu) ** 2).mean(1, keepdim=True)
                rs = 1 / torch.sqrt(var + 1e-5)
                want = (xf - mu) * rs * w.float() + b.float()
                if not (close(mean[rows], mu[:, 0], 1e-5, 1e-5) and close(rstd[rows], rs[:, 0], 1e-5, 1e-5)):
                    return False
            else:
                want = xf * (1 / torch.sqrt((xf * xf).mean(1, keepdim=True) + 1e-6)) * w.float()
            return close(y[rows], want, 1e-2, 1.6e-2)

        if kind == "layernorm":
            run = lambda s: ops.layernorm_kernel[(m,)](s[0], s[3], s[1], s[2], s[4], s[5], n, n, n, 1e-5, BLOCK=1024)  # noqa: E731
            run_host = lambda h: ops.layernorm(h[0], h[1], h[2], 1e-5)  # noqa: E731
        else:
            run = lambda s: ops.rmsnorm_kernel[(m,)](s[0], s[1], s[3], n, n, n, 1e-6, BLOCK=4096)  # noqa: E731
            run_host = lambda h: ops.rmsnorm(h[0], h[1], 1e-6)  # noqa: E731
        return dict(name=f"{kind}_bf16_{m_full}x{n}", kernel=kind, jit=getattr(ops, kind + "_kernel"), unit="GB/s", bound="hbm", dtype="bf16",
                    work=2 * m * n * 2, set_bytes=2 * m * n * 2, make=make, run=run, verify=verify, host=host, run_host=run_host)

    def gelu_wl():
        n_full = 1 << 28
        n = part(n_full, 1024)

        def verify(s):
            k = min(n, 1 << 22)
            return close(s[1][:k], torch.nn.functional.gelu(s[0][:k], approximate="tanh"), 1e-5, 1e-5) and \
                close(s[1][-k:], torch.nn.functional.gelu(s[0][-k:], approximate="tanh"), 1e-5, 1e-5)

        return dict(
            name="gelu_tanh_f32_2p28", kernel="gelu", jit=ops.tanh_gelu_kernel, unit="GB/s", bound="hbm", dtype="f32",
            work=2 * n * 4, set_bytes=2 * n * 4,
            make=lambda i: (torch.randn(n, device="cuda", generator=gen(i)) * 2, torch.empty(n, device="cuda")),
            run=lambda s: ops.tanh_gelu_kernel[(n // 1024,)](s[0], s[1], n, BLOCK=1024), verify=verify,
            host=lambda: ((np.random.default_rng(0).standard_normal(n // 8).astype(np.float32) * 2),),
            run_host=lambda h: ops.tanh_gelu(h[0]), host_units=2 * (n // 8) * 4)

    # ---- config 3: fused matmul fp16 ----
    def matmul_wl(m_full, n, k):
        m = part(m_full, 128)

        def make(i):
            g = gen(i)
            a = ((torch.rand(m, k, device="cuda", generator=g) * 2 - 1) / math.sqrt(k)).half()
            b = ((torch.rand(k, n, device="cuda", generator=g) * 2 - 1) / math.sqrt(k)).half()
            bias = (0.1 * torch.randn(n, device="cuda", generator=g)).half()
            return a, b, bias, torch.empty(m, n, device="cuda", dtype=torch.float16)

        def host():
            r = np.random.default_rng(0)
            sc = np.float32(1 / math.sqrt(k))
            return _f16_host((r.random((m, k), dtype=np.float32) * 2 - 1) * sc), \
                _f16_host((r.random((k, n), dtype=np.float32) * 2 - 1) * sc), \
                _f16_host(0.1 * r.standard_normal(n, dtype=np.float32))

        def verify(s):  # 64 rows against float32 matmul + erf-GELU in torch, float16 tolerance
            a, b, bias, c = s
            rows = torch.linspace(0, m - 1, 64, device="cuda").long()
            want = torch.nn.functional.gelu(a[rows].float() @ b.float() + bias.float())
            return close(c[rows], want, 1e-3, 2e-3)

        return dict(name=f"matmul_bias_gelu_f16_{m_full}x{n}x{k}", kernel="matmul", jit=ops.matmul_bias_gelu_kernel,
                    unit="TFLOP/s", bound="tensor",
                    dtype="f16", work=2 * m * n * k, set_bytes=(m * k + k * n + m * n) * 2, make=make,
                    run=lambda s: ops.matmul_bias_gelu(s[0], s[1], s[2], s[3]), verify=verify,
                    host=host, run_host=lambda h: ops.matmul_bias_gelu(h[0], h[1], h[2]))

    # ---- not a graded config: the reference's exact int8 matmul (benchmarks/bench_matmul.py:100-131) ----
    def int8_matmul_wl(m_full, n, k):
        m = part(m_full, 128)

        def make(i):
            g = gen(i)
            return (torch.randint(-128, 128, (m, k), device="cuda", dtype=torch.int8, generator=g),
                    torch.randint(-128, 128, (k, n), device="cuda", dtype=torch.int8, generator=g),
                    torch.empty(m, n, device="cuda", dtype=torch.int32))

        def verify(s):  # exact: 16 rows in float64 (|sum| < 2^53)
            rows = torch.linspace(0, m - 1, 16, device="cuda").long()
            want = (s[0][rows].double() @ s[1].double()).long()
            return bool((s[2][rows].long() == want).all())

        return dict(name=f"matmul_int8_{m_full}x{n}x{k}", kernel="matmul_int", jit=ops.int8_matmul_kernel, unit="TOP/s",
                    bound="tensor", peak_scale=2.0, dtype="s8", work=2 * m * n * k, set_bytes=m * k + k * n + 4 * m * n, make=make,
                    run=lambda s: ops.int_matmul(s[0], s[1], s[2]), verify=verify)

    # ---- config 4: attention bf16 [8, 32, 4096, 128] ----
    def attention_wl(causal):
        zf, hf, s_, d = 8, 32, 4096, 128
        bh = part(zf * hf)
        z, h = (zf, hf) if bh == zf * hf else (1, bh)

        def make(i):
            g = gen(i)
            q, k, v = (torch.randn(z, h, s_, d, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
            return q, k, v, torch.empty_like(q), torch.empty(z, h, s_, device="cuda")

        flops = 4 * z * h * s_ * s_ * d // (2 if causal else 1)
        zh = 2  # batches of the host (end-to-end) leg: a quarter of the workload, to bound the bench's run time

        def host():
            r = np.random.default_rng(0)
            return tuple(_bf16_host((zh, hf, s_, d), r) for _ in range(3))

        def verify(s):  # the last (batch, head) slice, 192 query rows, against float32 softmax(QK^T)V in torch
            q, k, v, o, _ = s
            rows = torch.cat([torch.arange(0, 64, device="cuda"), torch.linspace(64, s_ - 1, 128, device="cuda").long()])
            sc = (q[-1, -1, rows].float() @ k[-1, -1].float().T) / math.sqrt(d)
            if causal:
                sc = sc.masked_fill(torch.arange(s_, device="cuda")[None, :] > rows[:, None], float("-inf"))
            want = torch.softmax(sc, 1) @ v[-1, -1].float()
            return close(o[-1, -1, rows], want, 2e-2, 1.6e-2)

        return dict(name=f"attention_bf16_8x32x4096x128_{'causal' if causal else 'full'}", kernel="attention",
                    jit=ops.attention_kernel,
                    unit="TFLOP/s", bound="tensor", dtype="bf16", work=flops, set_bytes=4 * z * h * s_ * d * 2,
                    make=make, run=lambda s: ops.attention(s[0], s[1], s[2], causal, None, s[3]), verify=verify,
                    host=host, run_host=lambda hh: ops.attention(hh[0], hh[1], hh[2], causal),
                    host_units=4 * zh * hf * s_ * s_ * d // (2 if causal else 1))

    # ---- config 5: histogram / cumsum ----
    def hist_wl(kind):
        n_full = int((1 << 30) * scale)
        n = part(n_full, 4096)
        bins = 256 if kind == "uniform256" else 4096

        def make(i):
            g = gen(i)
            if kind == "uniform256":
                x = torch.randint(0, 256, (n,), device="cuda", dtype=torch.int32, generator=g)
            else:  # Zipf(1.1) clipped to 4095 by inverse CDF (same law as workloads.zipf_clipped)
                from scipy.special import zeta

                kk = np.arange(1, bins - 1, dtype=np.float64)
                cdf = torch.from_numpy(np.concatenate([[0.0], np.cumsum(kk ** -1.1 / zeta(1.1, 1))])).cuda()
                x = torch.empty(n, device="cuda", dtype=torch.int32)
                step = 1 << 26
                for s0 in range(0, n, step):
                    u = torch.rand(min(step, n - s0), device="cuda", generator=g, dtype=torch.float64)
                    x[s0 : s0 + step] = torch.searchsorted(cdf, u, right=True).clamp_(max=bins - 1).int()
            return x, torch.zeros(bins, device="cuda", dtype=torch.int32)

        def run(s):
            ops.histogram_kernel[(-(-n // 1024),)](s[0], s[1], n, 0.0, 1.0, NUM_BINS=bins, BLOCK=1024)
            if WORLD > 1:
                import torch.distributed as dist

                dist.all_reduce(s[1])

        def verify(s):
            # one fresh launch into zeroed bins; bit-exact against torch.bincount of the same data, summed over
            # the ranks exactly as the bins are (at N > 1 every rank must hold the global counts)
            s[1].zero_()
            run(s)
            want = torch.zeros(bins, device="cuda", dtype=torch.int64)
            for s0 in range(0, n, 1 << 28):
                want += torch.bincount(s[0][s0 : s0 + (1 << 28)], minlength=bins)
            total = torch.tensor([n], device="cuda", dtype=torch.int64)
            if WORLD > 1:
                import torch.distributed as dist

                dist.all_reduce(want)
                dist.all_reduce(total)
            # the bins are int32 and wrap like the reference's (hist = new_zeros(int32) + atomic_add): eight ranks' worth
            # of the Zipf tail bin is 3.5e9 counts, so the comparison is modulo 2^32
            return bool((s[1] == want.to(torch.int32)).all()) and (int(s[1].long().sum()) - int(total)) % (1 << 32) == 0

        return dict(name=f"histogram_i32_2p30_{kind}", kernel="histogram", jit=ops.histogram_kernel, unit="GB/s", bound="hbm", dtype="i32",
                    work=n * 4, set_bytes=n * 4, make=make, run=run, verify=verify, sets=1,
                    collective="all_reduce of the bins" if WORLD > 1 else None,
                    host=lambda: (np.random.default_rng(0).integers(0, bins, n // 16).astype(np.int32),),
                    run_host=lambda h: ops.histogram(h[0], bins, 0.0, float(bins)), host_units=(n // 16) * 4)

    def cumsum_wl(kind):
        n_full = int((1 << 30) * scale) if kind == "i32" else int((1 << 28) * scale)
        n = part(n_full, 4096)

        def make(i):
            g = gen(i)
            if kind == "i32":
                x = torch.randint(0, 16, (n,), device="cuda", dtype=torch.int32, generator=g)
            else:
                x = torch.randn(n, device="cuda", generator=g)
            return x, torch.empty_like(x)

        def run(s):
            if WORLD > 1:  # local total -> all-gather -> offset kernel -> seeded local scan (reads the shard twice)
                edist.sharded_cumsum(s[0], edist.cuda_total, lambda x, seed: _scan_into(x, s[1], seed))
            else:
                ops.cumsum_kernel[(1,)](s[1], s[0], 1, n, n, n, REVERSE=False, BLOCK_M=1, BLOCK_N=1 << 30)

        def _scan_into(x, out, seed):
            from enceladus_b200.runtime import interop

            N.call("enc_cumsum", x.data_ptr(), out.data_ptr(), 1, n, n, n, 0, interop.dtype_code(x),
                   seed.data_ptr(), -1, interop.current_stream())
            return out

        def verify(s):
            # differences of neighbouring outputs give back the input (every element), the first output is the input
            # plus the offset of the ranks before, and the last output of the last rank is the global total; all in
            # the scan's own arithmetic (int32 wraps; float32 within 1e-4 of the largest prefix)
            x, out = s
            import torch.distributed as dist

            if kind == "i32":
                ok = bool((out[1:] - out[:-1] == x[1:]).all())
                local = int(x.sum(dtype=torch.int64))
                before, total = 0, local
                if WORLD > 1:
                    sums = torch.zeros(WORLD, device="cuda", dtype=torch.int64)
                    sums[RANK] = local
                    dist.all_reduce(sums)
                    before, total = int(sums[:RANK].sum()), int(sums.sum())
                ok = ok and (int(out[0]) - before - int(x[0])) % (1 << 32) == 0
                ok = ok and (int(out[-1]) - before - local) % (1 << 32) == 0
                return ok and (RANK != WORLD - 1 or (int(out[-1]) - total) % (1 << 32) == 0)
            exact = torch.cumsum(x.double(), 0)
            if WORLD > 1:
                sums = torch.zeros(WORLD, device="cuda", dtype=torch.float64)
                sums[RANK] = exact[-1]
                dist.all_reduce(sums)
                exact += sums[:RANK].sum()
            scale_ = max(float(exact.abs().max()), 1.0)
            return bool(torch.isfinite(out).all()) and float((out.double() - exact).abs().max()) <= 1e-4 * scale_

        nh = n // 16
        return dict(name=f"cumsum_{kind}_{'2p30' if kind == 'i32' else '2p28'}", kernel="cumsum", jit=ops.cumsum_kernel, unit="GB/s",
                    bound="hbm", dtype=kind, work=2 * n * 4, set_bytes=2 * n * 4, make=make, run=run, verify=verify, sets=1,
                    collective="all_gather of one total per rank + offset kernel" if WORLD > 1 else None,
                    host=lambda: ((np.random.default_rng(0).integers(0, 16, nh).astype(np.int32),) if kind == "i32"
                                  else (np.random.default_rng(0).standard_normal(nh).astype(np.float32),)),
                    run_host=lambda h: ops.cumsum(h[0]), host_units=2 * nh * 4)

    W["layernorm"] = lambda: norm_wl("layernorm")
    W["softmax"] = softmax_wl
    W["softmax_4096x4096"] = lambda: softmax_wl(4096)  # the reference's own benchmark shape (benchmarks/bench_softmax.py)
    W["rmsnorm"] = lambda: norm_wl("rmsnorm")
    W["gelu"] = gelu_wl
    if N.num_variants(N.K_MATMUL) > 0:
        W["matmul_8192"] = lambda: matmul_wl(8192, 8192, 8192)
        W["matmul_4096x4096x16384"] = lambda: matmul_wl(4096, 4096, 16384)
        W["matmul_int8_8192"] = lambda: int8_matmul_wl(8192, 8192, 8192)
    if N.num_variants(N.K_ATTENTION) > 0:
        W["attention_full"] = lambda: attention_wl(False)
        W["attention_causal"] = lambda: attention_wl(True)
    W["histogram_uniform256"] = lambda: hist_wl("uniform256")
    W["histogram_zipf4096"] = lambda: hist_wl("zipf4096")
    W["cumsum_i32"] = lambda: cumsum_wl("i32")
    W["cumsum_f32"] = lambda: cumsum_wl("f32")
    return W


# workload key -> name of its row (and of its CPU leg in oracle/cpu_legs.py)
ROW_NAMES = {
    "layernorm": "layernorm_bf16_16384x4096", "softmax": "softmax_f32_4096x1024", "softmax_4096x4096": "softmax_f32_4096x4096",
    "rmsnorm": "rmsnorm_bf16_16384x4096", "gelu": "gelu_tanh_f32_2p28", "matmul_8192": "matmul_bias_gelu_f16_8192x8192x8192",
    "matmul_4096x4096x16384": "matmul_bias_gelu_f16_4096x4096x16384", "matmul_int8_8192": "matmul_int8_8192x8192x8192",
    "attention_full": "attention_bf16_8x32x4096x128_full", "attention_causal": "attention_bf16_8x32x4096x128_causal",
    "histogram_uniform256": "histogram_i32_2p30_uniform256", "histogram_zipf4096": "histogram_i32_2p30_zipf4096",
    "cumsum_i32": "cumsum_i32_2p30", "cumsum_f32": "cumsum_f32_2p28",
}
ROW_DTYPES = {"layernorm": "bf16", "rmsnorm": "bf16", "softmax": "f32", "softmax_4096x4096": "f32", "gelu": "f32",
              "matmul_8192": "f16", "matmul_4096x4096x16384": "f16", "attention_full": "bf16", "attention_causal": "bf16",
              "histogram_uniform256": "i32", "histogram_zipf4096": "i32", "cumsum_i32": "i32", "cumsum_f32": "f32"}


# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of this rank's GPU while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.proc = None
        self.lines: list[str] = []
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self) -> int:
        return len(self.lines)

    def stop(self) -> None:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, start: int = 0, end: int | None = None) -> dict:
        rows = [ln.split(", ") for ln in self.lines[start:end] if ln.count(",") >= 6]
        if not rows:
            rows = [ln.split(", ") for ln in self.lines if ln.count(",") >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = sorted(float(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].strip() == "Active" for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][1]), "reasons": reasons,
                "samples": len(rows), "power_w_max": max(float(r[2]) for r in rows if r[2].replace(".", "").isdigit())}


class NvmlSampler:
    """The same readings taken through NVML from a thread of this process, about every millisecond, so that a timed
    region of a few milliseconds holds several samples (nvidia-smi cannot poll faster than every 100 ms).  Read-only:
    SM clock, its maximum, power draw and the clock event reasons."""

    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int, period_s: float = 0.001) -> None:
        import pynvml

        self.nv = pynvml
        pynvml.nvmlInit()
        self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
        self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        self.bits = (pynvml.nvmlClocksEventReasonHwSlowdown, pynvml.nvmlClocksEventReasonHwThermalSlowdown,
                     pynvml.nvmlClocksEventReasonSwThermalSlowdown, pynvml.nvmlClocksEventReasonSwPowerCap)
        self._read_once()  # fail here, not in the thread, if a query is not supported
        self.rows: list[tuple[float, float, int]] = []
        self.period = period_s
        self.running = True
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def _read_once(self) -> tuple[float, float, int]:
        nv = self.nv
        return (float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)), nv.nvmlDeviceGetPowerUsage(self.h) / 1e3,
                int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)))

    def _loop(self) -> None:
        while self.running:
            try:
                self.rows.append(self._read_once())
            except Exception:  # noqa: BLE001 - a failed query must not end the run; the summary shows fewer samples
                pass
            time.sleep(self.period)

    def mark(self) -> int:
        return len(self.rows)

    def stop(self) -> None:
        self.running = False
        self.thread.join(timeout=2)
        try:
            self.nv.nvmlShutdown()
        except Exception:  # noqa: BLE001
            pass

    def summary(self, start: int = 0, end: int | None = None) -> dict:
        rows = self.rows[start:end] or self.rows
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        sm = sorted(r[0] for r in rows)
        reasons = [n for n, b in zip(self.NAMES, self.bits) if any(r[2] & b for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons, "samples": len(rows),
                "power_w_max": max(r[1] for r in rows), "how": "NVML, about 1 ms apart"}


def make_sampler(index: int):
    """NVML from this process when it is there, the nvidia-smi poller otherwise."""
    try:
        return NvmlSampler(index)
    except Exception:  # noqa: BLE001 - no pynvml, no NVML, an unsupported query
        return ClockSampler(index)


def visible_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v for v in vis.split(",") if v.strip() != ""]
        try:
            return int(ids[local_rank])
        except (ValueError, IndexError):
            return local_rank
    return local_rank


def timed_region(run, sets, steps: int, warmup: int, graph: bool = True):
    """W warm-up steps, then exactly K steps between two events; returns ms per step (max over ranks).

    The K steps are captured into one CUDA graph and replayed, so that host launch latency (a few
    microseconds per launch through Python) does not hide kernels that run for about as long.
    """
    import torch

    for i in range(warmup):
        run(sets[i % len(sets)])
    torch.cuda.synchronize()
    g = None
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(steps):
                run(sets[(warmup + i) % len(sets)])
        g.replay()  # untimed: uploads the graph
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if g is not None:
        g.replay()
    else:
        for i in range(steps):
            run(sets[(warmup + i) % len(sets)])
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return max_over_ranks(e0.elapsed_time(e1)) / steps


def barrier():
    if WORLD > 1:
        import torch.distributed as dist

        dist.barrier()


def max_over_ranks(v: float) -> float:
    if WORLD > 1:
        import torch
        import torch.distributed as dist

        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return v


def sum_over_ranks(v: float) -> float:
    if WORLD > 1:
        import torch
        import torch.distributed as dist

        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t)
        return float(t.item())
    return v


def all_ranks(ok: bool) -> bool:
    return max_over_ranks(0.0 if ok else 1.0) == 0.0


def interop_view(a):
    """A torch CPU tensor over a NumPy array's memory (bfloat16 included)."""
    from enceladus_b200.runtime import interop

    return interop._np_as_torch_view(a)


def pinned(arrays):
    """Copies of NumPy arrays that live in pinned host memory (views of pinned torch tensors)."""
    import torch

    from enceladus_b200.runtime import interop

    out = []
    for a in arrays:
        t = torch.empty(a.shape, dtype=interop._np_as_torch_view(a).dtype, pin_memory=True)
        t.copy_(interop._np_as_torch_view(a))
        v = t.view(torch.uint16).numpy().view(a.dtype) if str(a.dtype) == "bfloat16" else t.numpy()
        out.append(v)
    return tuple(out)


def measure_pcie(nbytes: int = 256 << 20, reps: int = 4) -> dict:
    """Pinned host<->device copy bandwidth of this rank's GPU, GB/s: host-to-device alone, device-to-host alone,
    and both directions at once on two streams.  With N ranks every rank copies at the same time (barrier first),
    so the figure is what a rank gets while its neighbours load the same host: the roofline of the `e2e` leg."""
    import torch

    h_in = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    h_out = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    d_in = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    d_out = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return max_over_ranks(e0.elapsed_time(e1)) / reps * 1e-3

    def both():
        cur = torch.cuda.current_stream()
        s1.wait_stream(cur)
        s2.wait_stream(cur)
        with torch.cuda.stream(s1):
            d_in.copy_(h_in, non_blocking=True)
        with torch.cuda.stream(s2):
            h_out.copy_(d_out, non_blocking=True)
        cur.wait_stream(s1)
        cur.wait_stream(s2)

    t_h2d = timed(lambda: d_in.copy_(h_in, non_blocking=True))
    t_d2h = timed(lambda: h_out.copy_(d_out, non_blocking=True))
    t_both = timed(both)
    return {"h2d_gbs": nbytes / t_h2d / 1e9, "d2h_gbs": nbytes / t_d2h / 1e9,
            "duplex_gbs_each_way": nbytes / t_both / 1e9, "bytes": nbytes, "ranks_copying_at_once": WORLD,
            "how": "pinned torch tensors, copy_(non_blocking) on this rank's GPU, CUDA events, slowest rank"}


def bench_workload(wl: dict, steps: int, warmup: int, pk: dict, pk_kind: str, sampler, e2e: bool, pcie: dict | None,
                   min_region_ms: float = 0.0):
    """One bench row.  `min_region_ms` > 0 (per-kernel rows only, never the headline) raises `steps` until the
    timed region lasts about that long: a graph replay costs several microseconds to launch, which ten steps of
    a 7-microsecond kernel do not amortise."""
    import torch

    nsets = wl.get("sets") or max(1, min(16, -(-ROTATE_BYTES // wl["set_bytes"])))
    if wl["set_bytes"] * 2 > ROTATE_BYTES:
        nsets = wl.get("sets") or 2
    sets = [wl["make"](1000 * RANK + i) for i in range(nsets)]
    torch.cuda.synchronize()
    m0 = sampler.mark() if sampler else 0
    graph = USE_GRAPH and not (WORLD > 1 and wl["kernel"] in ("histogram", "cumsum"))  # collectives stay eager
    if min_region_ms > 0:
        wl["run"](sets[0])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        wl["run"](sets[-1])
        e1.record()
        torch.cuda.synchronize()
        est = max(max_over_ranks(e0.elapsed_time(e1)), 1e-3)
        steps = max(steps, min(200, int(min_region_ms / est) + 1))
    ms = timed_region(wl["run"], sets, steps, warmup, graph)
    if min_region_ms > 0 and graph and ms * steps < min_region_ms:
        # the estimate above is one EAGER launch, tens of microseconds of host time for a kernel of a few: size the
        # graph from the device time just measured and time again
        steps = min(1000, int(min_region_ms / max(ms, 1e-4)) + 1)
        ms = timed_region(wl["run"], sets, steps, warmup, graph)
    m1 = sampler.mark() if sampler else 0
    div = 1e9 if wl["unit"] == "GB/s" else 1e12
    achieved = wl["work"] / (ms * 1e-3) / div        # this rank's work over the slowest rank's time
    total = sum_over_ranks(wl["work"]) / (ms * 1e-3) / div
    peak = pk["hbm_gbs"] if wl["bound"] == "hbm" else pk["bf16_tflops"] * wl.get("peak_scale", 1.0)
    if "peak_scale" in wl:  # no int8 GEMM was measured on this pool: the 8-bit rate of the tensor cores is twice the 16-bit one
        pk_kind = f"{wl['peak_scale']:g} x {pk_kind} bf16"
    verify_error = None
    try:
        wl["run"](sets[0])
        ok = bool(wl["verify"](sets[0]))
    except Exception as e:  # noqa: BLE001 - a checker that cannot run is a failed check, not a failed bench
        ok = False
        verify_error = f"{type(e).__name__}: {e}"
    verified = all_ranks(ok)
    row = {
        "name": wl["name"], "value": total, "unit": wl["unit"], "ms_per_step": ms, "steps": steps,
        "warmup": warmup, "dtype": wl["dtype"], "buffer_sets": nsets, "cuda_graph": graph, "verified": verified,
        "roofline": {"bound": wl["bound"], "achieved": achieved, "peak": peak, "unit": wl["unit"],
                     "frac": achieved / peak, "peak_source": pk_kind, "traffic": NCU_TRAFFIC.get(wl["name"])},
    }
    if wl.get("collective"):
        row["collective_in_timed_region"] = wl["collective"]
    if verify_error:
        row["verify_error"] = verify_error
    if sampler:
        row["clocks"] = sampler.summary(m0, m1)
    del sets
    torch.cuda.empty_cache()
    if e2e and "run_host" in wl:
        h = pinned(wl["host"]())
        units = wl.get("host_units", wl["work"])
        # warm-up: the launch path keeps two page-locked output buffers alive in turn (the previous
        # result and the new one); both must exist before timing, page-locking 100+ MB takes tens of ms
        res = None
        for _ in range(3):
            res = wl["run_host"](h)
        barrier()
        torch.cuda.synchronize()
        reps = 3
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            res = wl["run_host"](h)
        e1.record()
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) / reps
        dev_ms = max_over_ranks(max(e0.elapsed_time(e1) / reps, wall * 1e3))
        last = wl["jit"].last_launch
        res = res if isinstance(res, tuple) else (res,)
        h2d, d2h = int(last.get("h2d_bytes", 0)), int(sum(r.nbytes for r in res))
        row["e2e"] = {"value": sum_over_ranks(units) / (dev_ms * 1e-3) / div, "unit": wl["unit"],
                      "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": dev_ms,
                      "workload_fraction": units / wl["work"]}
        # the host-array result must be what the same call returns for device-resident copies of the same inputs: bit for
        # bit (the staged pieces are independent), except the chained float32 scan, whose additions are ordered differently
        try:
            dev_in = tuple(interop_view(a).cuda() for a in h)
            want = wl["run_host"](dev_in)
            want = want if isinstance(want, tuple) else (want,)
            torch.cuda.synchronize()
            same = True
            for g, w in zip(res, want):
                gt, wt = interop_view(np.ascontiguousarray(g)), w.cpu().contiguous()
                if wl["kernel"] == "cumsum" and gt.dtype.is_floating_point:
                    same = same and bool((gt.double() - wt.double()).abs().max() <= 1e-4 * wt.double().abs().max())
                else:
                    same = same and gt.shape == wt.shape and bool(torch.equal(gt.view(torch.uint8), wt.view(torch.uint8)))
            del dev_in, want
        except Exception as e:  # noqa: BLE001 - reported, not fatal
            same = False
            row["e2e"]["verify_error"] = f"{type(e).__name__}: {e}"
        row["e2e"]["verified"] = all_ranks(same)
        if pcie:  # the copies alone, both directions overlapped, at the bandwidths measured in this run
            floor_ms = max(h2d / pcie["h2d_gbs"], d2h / pcie["d2h_gbs"], (h2d + d2h) / 2 / pcie["duplex_gbs_each_way"]) / 1e6
            row["e2e"]["pcie_floor_ms"] = floor_ms
            row["e2e"]["frac"] = floor_ms / dev_ms
    return row


def reference_shape_rows(pk: dict) -> list[dict]:
    """The shapes of the reference's own benchmark reports, so that its published numbers (Apple M4 Pro, Metal;
    benchmarks/results/2026-09-27-applegpu_g16s-2.md) have like-for-like rows.  Device-resident inputs, same
    timing as every other row; not graded configurations and no roofline claim beyond the fraction."""
    import torch

    from enceladus_b200 import ops

    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(1234 + RANK)
    rows = []

    def timed(name, unit, work, bound, make, run, published, nsets=None):
        set_bytes = sum(t.numel() * t.element_size() for t in make())
        nsets = nsets or max(2, min(16, -(-ROTATE_BYTES // max(set_bytes, 1))))
        sets = [make() for _ in range(nsets)]
        run(sets[0])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run(sets[-1])
        e1.record()
        torch.cuda.synchronize()
        steps = max(10, min(200, int(1.0 / max(e0.elapsed_time(e1), 1e-3)) + 1))
        ms = timed_region(run, sets, steps, 3, USE_GRAPH)
        if USE_GRAPH and ms * steps < 1.0:  # size the graph from the device time (the estimate was one eager launch)
            steps = min(1000, int(1.0 / max(ms, 1e-4)) + 1)
            ms = timed_region(run, sets, steps, 3, USE_GRAPH)
        value = work / (ms * 1e-3) / (1e9 if unit == "GB/s" else 1e12)
        peak = pk["hbm_gbs"] if bound == "hbm" else pk["bf16_tflops"] * (2.0 if unit == "TOP/s" else 1.0)
        rows.append({"name": name, "value": round(value, 1), "unit": unit, "ms_per_step": round(ms, 5),
                     "frac_of_peak": round(value / peak, 3), "published_m4pro": published})
        del sets
        torch.cuda.empty_cache()

    def randn(*shape, dt=torch.float32):
        return torch.randn(*shape, device=dev, generator=g).to(dt)

    m = n = 4096
    for dt, name, pub in ((torch.float32, "f32", 241.9), (torch.float16, "f16", 256.3)):
        timed(f"softmax_{name}_4096x4096", "GB/s", 2 * m * n * dt.itemsize, "hbm", lambda: (randn(m, n, dt=dt) * 4, torch.empty(m, n, device=dev, dtype=dt)),
              lambda s: ops.softmax_kernel[(m,)](s[1], s[0], n, n, n, BLOCK=n), pub)
    for dt, name, pl, pr in ((torch.float32, "f32", 237.4, 239.5), (torch.float16, "f16", 241.9, 247.4)):
        mk = lambda: (randn(m, n, dt=dt), randn(n, dt=dt), randn(n, dt=dt), torch.empty(m, n, device=dev, dtype=dt),  # noqa: E731
                      torch.empty(m, device=dev), torch.empty(m, device=dev))
        timed(f"layernorm_{name}_4096x4096", "GB/s", 2 * m * n * dt.itemsize, "hbm", mk,
              lambda s: ops.layernorm_kernel[(m,)](s[0], s[3], s[1], s[2], s[4], s[5], n, n, n, 1e-5, BLOCK=n), pl)
        timed(f"rmsnorm_{name}_4096x4096", "GB/s", 2 * m * n * dt.itemsize, "hbm", mk,
              lambda s: ops.rmsnorm_kernel[(m,)](s[0], s[1], s[3], n, n, n, 1e-6, BLOCK=n), pr)
    na = 1 << 26
    timed("vector_add_f32_2p26", "GB/s", 3 * na * 4, "hbm", lambda: (randn(na), randn(na), torch.empty(na, device=dev)),
          lambda s: ops.add_kernel[(na // 1024,)](s[0], s[1], s[2], na, BLOCK=1024), 236.6)
    timed("row_cumsum_f32_4096x4096", "GB/s", 2 * m * n * 4, "hbm", lambda: (randn(m, n), torch.empty(m, n, device=dev)),
          lambda s: ops.cumsum_kernel[(m,)](s[1], s[0], m, n, n, n, REVERSE=False, BLOCK_M=1, BLOCK_N=n), 242.2)
    nh = 1 << 24
    for bins, pub in ((64, 31.1), (4096, 62.5)):
        timed(f"histogram_f32_2p24_{bins}bins", "GB/s", nh * 4, "hbm", lambda: (torch.rand(nh, device=dev, generator=g), torch.zeros(bins, device=dev, dtype=torch.int32)),
              lambda s: ops.histogram_kernel[(nh // 1024,)](s[0], s[1], nh, 0.0, float(bins), NUM_BINS=bins, BLOCK=1024), pub)
    for (mm, nn, kk), pub in (((4096, 4096, 4096), 6.04), ((2000, 2000, 2000), 5.86), ((513, 513, 513), 4.31), ((1024, 4096, 1024), 6.03)):
        mk = lambda: (randn(mm, kk, dt=torch.float16) / math.sqrt(kk), randn(kk, nn, dt=torch.float16), randn(nn, dt=torch.float16) * 0.1,  # noqa: E731
                      torch.empty(mm, nn, device=dev, dtype=torch.float16))
        timed(f"matmul_f16_{mm}x{nn}x{kk}", "TFLOP/s", 2 * mm * nn * kk, "tensor", mk, lambda s: ops.matmul_desc(s[0], s[1], s[3]), pub, nsets=4)
        if mm == 4096:
            timed("matmul_bias_gelu_f16_4096x4096x4096", "TFLOP/s", 2 * mm * nn * kk, "tensor", mk,
                  lambda s: ops.matmul_bias_gelu(s[0], s[1], s[2], s[3]), 6.00, nsets=4)
    timed("matmul_int8_4096x4096x4096", "TOP/s", 2 * 4096**3, "tensor",
          lambda: (torch.randint(-128, 128, (4096, 4096), device=dev, dtype=torch.int8, generator=g),
                   torch.randint(-128, 128, (4096, 4096), device=dev, dtype=torch.int8, generator=g),
                   torch.empty(4096, 4096, device=dev, dtype=torch.int32)),
          lambda s: ops.int_matmul(s[0], s[1], s[2]), 4.75, nsets=4)
    for (seq, d), (pn, pc) in (((4096, 128), (5.04, 4.93)), ((4096, 64), (5.26, 5.06)), ((2048, 128), (5.23, None)), ((2048, 64), (4.83, None))):
        mk = lambda: (*(randn(1, 16, seq, d, dt=torch.float16) for _ in range(3)), torch.empty(1, 16, seq, d, device=dev, dtype=torch.float16))  # noqa: E731
        for causal, pub in ((False, pn), (True, pc)):
            if pub is None and causal:
                continue
            timed(f"attention_f16_1x16x{seq}x{d}_{'causal' if causal else 'full'}", "TFLOP/s", 4 * 16 * seq * seq * d // (2 if causal else 1), "tensor",
                  mk, lambda s: ops.attention(s[0], s[1], s[2], causal, None, s[3]), pub, nsets=8)
    return rows


# ---------------------------------------------------------------------------------------------------
# CPU baselines (the reference's own CPU path; oracle/cpu_legs.py).  Run before CUDA is initialised, because
# the legs fork worker processes.
def cpu_baselines(names: list[str], headline: str, headline_budget: float, row_budget: float) -> dict[str, dict]:
    from oracle import cpu_legs

    out = {}
    for n in names:
        if n not in cpu_legs.LEGS:
            continue
        try:
            b = cpu_legs.baseline(n, headline_budget if n == headline else row_budget,
                                  numpy_budget_s=2.0 if n == headline else 0.5)
        except Exception as e:  # noqa: BLE001 - a failing CPU leg must not stop the GPU measurement
            b = {"error": f"{type(e).__name__}: {e}"}
        if b is not None:
            out[n] = b
    return out


def reference_arm(args) -> None:
    """`--impl reference`: the reference's own CPU implementation of the headline workload (its interpreter, from
    oracle/_ref) on all host cores, rank 0 only.  Each step runs one bounded sample of the workload."""
    if RANK != 0:
        return
    from oracle import cpu_legs

    name = ROW_NAMES.get(args.workload, args.workload)
    if name not in cpu_legs.LEGS:
        print(json.dumps({"impl": "reference", "unavailable": f"no CPU leg for workload {name}"}))
        return
    r = cpu_legs.Runner(name, budget_s=0.4)  # about 0.4 s of all-core work per step
    try:
        samples = []
        for i in range(args.warmup + args.steps):
            dt, units = r.step()
            if i >= args.warmup:
                samples.append((dt, units))
        dt = sum(s[0] for s in samples)
        units = sum(s[1] for s in samples)
        scale = 1e9 if r.leg.unit == "GB/s" else 1e12
        value = units / dt / scale
        full_units = r.leg.units(None, 0, r.leg.full_pieces)
        workers = r.workers if r.leg.parallel else cpu_legs.blas_threads()
        line = {"impl": "reference",
                "metric": f"{name} algorithmic {'HBM GB/s (read+write)' if r.leg.unit == 'GB/s' else r.leg.unit}",
                "value": value, "unit": r.leg.unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": full_units / (value * scale) * 1e3, "higher_is_better": True, "scaling": args.scaling,
                "vs_baseline": None, "dtype": ROW_DTYPES.get(args.workload), "data": "synthetic",
                "config": {"workload": name},
                "cpu_baseline": {"value": value, "unit": r.leg.unit, "cores": workers, "kind": r.kind,
                                 "sample": "each step: " + r.sample() + f"; {len(samples)} timed steps, {dt:.2f} s; "
                                           "ms_per_step is the whole workload at this rate"},
                "e2e": {"value": value, "unit": r.leg.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
    finally:
        r.close()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="layernorm")
    ap.add_argument("--kernels", default="all", help="per-kernel rows: all, none, or a comma list")
    ap.add_argument("--kernel-steps", type=int, default=10)
    ap.add_argument("--scale", type=float, default=1.0, help="shrinks the 2^30 / 2^28 element workloads")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="N > 1: weak = the whole configuration on every rank, strong = the configuration cut into N shards")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch the timed steps eagerly instead of as one CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-baseline-headline-only", action="store_true")
    ap.add_argument("--no-reference-shapes", action="store_true", help="skip the rows at the reference's own benchmark shapes")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    global USE_GRAPH
    USE_GRAPH = not args.no_graph

    if args.impl == "reference":
        reference_arm(args)
        return
    if args.workload not in ROW_NAMES:
        raise SystemExit(f"unknown workload {args.workload!r}; choose from {sorted(ROW_NAMES)}")
    row_keys = ([] if args.kernels == "none" else [k for k in ROW_NAMES if k != args.workload] if args.kernels == "all"
                else [k for k in args.kernels.split(",") if k != args.workload])

    # ---- CPU baselines first: N = 1, rank 0, before this process touches CUDA (the legs fork workers) ----
    cpu = {}
    if WORLD == 1 and not args.no_cpu_baseline:
        keys = [args.workload] + ([] if args.cpu_baseline_headline_only else row_keys)
        cpu = cpu_baselines([ROW_NAMES[k] for k in keys if k in ROW_NAMES], ROW_NAMES[args.workload], 6.0, 1.5)

    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(LOCAL_RANK)
    if WORLD > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", LOCAL_RANK))
    from enceladus_b200 import _native as N

    N.load()
    pk, pk_kind = peaks()
    strong = args.scaling == "strong" and WORLD > 1
    W = workloads(args.scale, (RANK, WORLD) if strong else None)
    if args.workload not in W:
        raise SystemExit(f"workload {args.workload!r} is not available in this build; choose from {sorted(W)}")
    sampler = make_sampler(visible_gpu_index(LOCAL_RANK)) if RANK == 0 else None
    time.sleep(0.3)
    pcie = None if args.no_e2e else measure_pcie()

    head = bench_workload(W[args.workload](), args.steps, args.warmup, pk, pk_kind, sampler, e2e=not args.no_e2e, pcie=pcie)
    rows = []
    launches = args.steps
    for k in row_keys:
        if k not in W:
            continue
        try:
            rows.append(bench_workload(W[k](), args.kernel_steps, 3, pk, pk_kind, sampler, e2e=not args.no_e2e, pcie=pcie,
                                       min_region_ms=1.0))
            launches += rows[-1]["steps"]
        except Exception as e:  # noqa: BLE001 - one failing workload must not hide the others
            rows.append({"name": ROW_NAMES.get(k, k), "error": f"{type(e).__name__}: {e}"})
            torch.cuda.empty_cache()
    ref_rows = []
    if args.kernels == "all" and not args.no_reference_shapes:
        try:
            ref_rows = reference_shape_rows(pk)
        except Exception as e:  # noqa: BLE001 - extra rows must not hide the graded ones
            ref_rows = [{"error": f"{type(e).__name__}: {e}"}]
    if sampler:
        sampler.stop()
    if WORLD > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    if RANK != 0:
        return

    def compact(r: dict) -> dict:
        if "error" in r:
            return {"error": r["error"]}
        c = {"value": round(r["value"], 2), "unit": r["unit"], "frac": round(r["roofline"]["frac"], 4),
             "ms_per_step": round(r["ms_per_step"], 5), "steps": r["steps"], "verified": r["verified"],
             "e2e_value": round(r["e2e"]["value"], 2) if "e2e" in r else None,
             "e2e_frac": round(r["e2e"]["frac"], 3) if "e2e" in r and "frac" in r["e2e"] else None,
             "e2e_verified": r["e2e"].get("verified") if "e2e" in r else None}
        if r.get("collective_in_timed_region"):
            c["collective"] = r["collective_in_timed_region"]
        if r.get("verify_error"):
            c["verify_error"] = r["verify_error"]
        b = cpu.get(r["name"])
        if b and "value" in b:
            c["cpu"] = {"value": round(b["value"], 5), "cores": b["cores"], "kind": b["kind"],
                        "numpy_reference": round(b.get("numpy_reference", {}).get("value", 0.0), 5) or None}
        return c

    roofline = dict(head["roofline"])
    roofline["per_kernel"] = {r["name"]: compact(r) for r in [head, *rows]}
    e2e = head.get("e2e")
    if e2e is not None and pcie is not None:
        e2e = dict(e2e, pcie=pcie)
    # key order matters to a reader who keeps only the end of the line: the rows at the reference's own shapes and
    # the long CPU-sample descriptions come first, the graded per-kernel map last
    line = {
        "metric": f"{head['name']} algorithmic {'HBM GB/s (read+write)' if head['unit'] == 'GB/s' else head['unit']}",
        "reference_shapes": ref_rows,
        "cpu_baselines": {k: v for k, v in cpu.items() if k != head["name"]},
        "run": {"l2": f"rotating {head['buffer_sets']} buffer sets (> 4x L2 in total)",
                "sharding": ("the configuration cut into contiguous shards, one per rank" if strong else
                             "same per-GPU workload on every rank") + "; no data-path collective except the histogram's "
                            "all-reduce of bins and the cumsum's all-gather of totals",
                "timed_region": "K launches captured in one CUDA graph" if head.get("cuda_graph") else "K eager launches"},
        "value": head["value"], "unit": head["unit"], "n_gpus": WORLD, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
        "dtype": head["dtype"], "data": "synthetic", "config": {"workload": head["name"]},
        "verified": head["verified"], "clocks": head.get("clocks"), "gpu_launches": launches,
        "e2e": e2e, "cpu_baseline": cpu.get(head["name"]), "roofline": roofline,
    }
    print(json.dumps(line))


if __name__ == "__main__":
    main()
