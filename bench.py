"""Benchmark of the kernel set on B200: per-kernel HBM GB/s or TFLOP/s against the measured roofline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--kernels all|none|a,b,...]
                    [--impl ours|reference] [--cpu-baseline-all] [--no-e2e]

Prints ONE JSON line.  The headline workload (default `layernorm`: LayerNorm over bf16 [16384, 4096]) is
timed for exactly K steps after W warm-up steps; `per_kernel` carries one row for every other workload
of the kernel set, each timed the same way with fewer steps.  A step is one launch of the kernel over
one batch of seeded synthetic input that is already resident in HBM.  Between steps the kernels rotate
through several buffer sets whose total size exceeds L2 several times, so every step reads from DRAM.

  value      algorithmic bytes (or FLOPs) of all ranks / device time (CUDA events, max over ranks)
  e2e        the same metric through the public launch path with HOST (pinned NumPy) arguments:
             host->device copy, kernel, device->host copy inside the timed region
  roofline   achieved / measured peak (MEASURED_PEAKS.json if present, else the stated fallback)
  cpu_baseline   the NumPy restatement of the reference's CPU path on this host's cores, bounded sample

N > 1 (under torchrun): every rank runs the same per-GPU workload on its own shard (weak scaling);
histogram adds its all-reduce of the bins and the flat cumsum its all-gather of shard totals inside the
timed region.  `--impl reference` times the CPU restatement of the reference with all host threads.
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
from concurrent.futures import ThreadPoolExecutor
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
    "layernorm_bf16_16384x4096": 216_550_656,       # profiles/layernorm.md
    "rmsnorm_bf16_16384x4096": 217_106_176,         # profiles/rmsnorm.md
    "softmax_f32_4096x1024": 16_793_600,            # profiles/softmax.md (the 16 MiB output stays in L2)
    "gelu_tanh_f32_2p28": 2_100_776_000,            # profiles/gelu.md
    "histogram_i32_2p30_uniform256": 8 * 540_655_616,   # profiles/hist_uniform256.md, captured at 2^27
    "histogram_i32_2p30_zipf4096": 8 * 540_067_328,     # profiles/hist_zipf4096.md, captured at 2^27
    "cumsum_i32_2p30": 8 * 1_014_728_192,           # profiles/cumsum_i32.md, captured at 2^27
    "cumsum_f32_2p28": 2 * 1_016_665_600,           # profiles/cumsum_f32.md, captured at 2^27
    "matmul_bias_gelu_f16_8192x8192x8192": 1_109_306_624,   # profiles/matmul.md
    "matmul_int8_8192x8192x8192": 571_891_712,              # profiles/matmul_int8.md
    "attention_bf16_8x32x4096x128_full": 1_052_659_968,     # profiles/attention_full.md
    "attention_bf16_8x32x4096x128_causal": 1_057_350_912,   # profiles/attention_causal.md
}


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
# Workloads.  Each returns a dict with: make(dev, i) -> argument set number i on the device, run(set),
# work (algorithmic bytes or flops per launch), unit, bound, dtype, and optionally host()/run_host()
# for the end-to-end path and cpu() for the CPU baseline.
# ---------------------------------------------------------------------------------------------------
def _bf16_host(shape, rng, scale=1.0, shift=0.0):
    import ml_dtypes

    return (shift + scale * rng.standard_normal(shape)).astype(np.float32).astype(ml_dtypes.bfloat16)


def workloads(scale: float = 1.0):
    import torch

    from enceladus_b200 import _native as N
    from enceladus_b200 import ops
    from oracle import enceladus_oracle as O  # CPU baseline leg only

    W = {}

    def gen(seed):
        g = torch.Generator(device="cuda")
        g.manual_seed(seed)
        return g

    # ---- config 1: softmax fp32 [4096, 1024] ----
    def softmax_wl(n=1024):
        m = 4096
        return dict(
            name=f"softmax_f32_4096x{n}", kernel="softmax", jit=ops.softmax_kernel, unit="GB/s", bound="hbm", dtype="f32",
            work=2 * m * n * 4, set_bytes=2 * m * n * 4,
            make=lambda i: (torch.randn(m, n, device="cuda", generator=gen(i)) * 4, torch.empty(m, n, device="cuda")),
            run=lambda s: ops.softmax_kernel[(m,)](s[1], s[0], n, n, n, BLOCK=n),
            host=lambda: (np.random.default_rng(0).standard_normal((m, n)).astype(np.float32) * 4,),
            run_host=lambda h: ops.softmax(h[0]),
            cpu=lambda h: O.softmax(h[0]), cpu_units=2 * m * n * 4)

    # ---- config 2: LayerNorm / RMSNorm bf16 [16384, 4096], tanh-GELU fp32 2^28 ----
    def norm_wl(kind):
        m, n = 16384, 4096

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

        if kind == "layernorm":
            run = lambda s: ops.layernorm_kernel[(m,)](s[0], s[3], s[1], s[2], s[4], s[5], n, n, n, 1e-5, BLOCK=1024)  # noqa: E731
            run_host = lambda h: ops.layernorm(h[0], h[1], h[2], 1e-5)  # noqa: E731
            cpu = lambda h, rows=None: O.layernorm(h[0][:rows], h[1], h[2], 1e-5)  # noqa: E731
        else:
            run = lambda s: ops.rmsnorm_kernel[(m,)](s[0], s[1], s[3], n, n, n, 1e-6, BLOCK=4096)  # noqa: E731
            run_host = lambda h: ops.rmsnorm(h[0], h[1], 1e-6)  # noqa: E731
            cpu = lambda h, rows=None: O.rmsnorm(h[0][:rows], h[1], 1e-6)  # noqa: E731
        return dict(name=f"{kind}_bf16_16384x4096", kernel=kind, jit=getattr(ops, kind + "_kernel"), unit="GB/s", bound="hbm", dtype="bf16",
                    work=2 * m * n * 2, set_bytes=2 * m * n * 2, make=make, run=run, host=host, run_host=run_host,
                    cpu=cpu, cpu_rows=m, cpu_units=2 * m * n * 2, rows=m, row_bytes=2 * n * 2)

    def gelu_wl():
        n = 1 << 28
        return dict(
            name="gelu_tanh_f32_2p28", kernel="gelu", jit=ops.tanh_gelu_kernel, unit="GB/s", bound="hbm", dtype="f32",
            work=2 * n * 4, set_bytes=2 * n * 4,
            make=lambda i: (torch.randn(n, device="cuda", generator=gen(i)) * 2, torch.empty(n, device="cuda")),
            run=lambda s: ops.tanh_gelu_kernel[(n // 1024,)](s[0], s[1], n, BLOCK=1024),
            host=lambda: ((np.random.default_rng(0).standard_normal(n // 8).astype(np.float32) * 2),),
            run_host=lambda h: ops.tanh_gelu(h[0]), host_units=2 * (n // 8) * 4,
            cpu=lambda h: O.gelu_tanh(h[0]), cpu_units=2 * (n // 8) * 4)

    # ---- config 3: fused matmul fp16 ----
    def matmul_wl(m, n, k):
        def make(i):
            g = gen(i)
            a = ((torch.rand(m, k, device="cuda", generator=g) * 2 - 1) / math.sqrt(k)).half()
            b = ((torch.rand(k, n, device="cuda", generator=g) * 2 - 1) / math.sqrt(k)).half()
            bias = (0.1 * torch.randn(n, device="cuda", generator=g)).half()
            return a, b, bias, torch.empty(m, n, device="cuda", dtype=torch.float16)

        def host():
            r = np.random.default_rng(0)
            sc = np.float32(1 / math.sqrt(k))
            return ((r.random((m, k), dtype=np.float32) * 2 - 1) * sc).astype(np.float16), \
                   ((r.random((k, n), dtype=np.float32) * 2 - 1) * sc).astype(np.float16), \
                   (0.1 * r.standard_normal(n, dtype=np.float32)).astype(np.float16)

        return dict(name=f"matmul_bias_gelu_f16_{m}x{n}x{k}", kernel="matmul", jit=ops.matmul_bias_gelu_kernel,
                    unit="TFLOP/s", bound="tensor",
                    dtype="f16", work=2 * m * n * k, set_bytes=(m * k + k * n + m * n) * 2, make=make,
                    run=lambda s: ops.matmul_bias_gelu(s[0], s[1], s[2], s[3]),
                    host=host, run_host=lambda h: ops.matmul_bias_gelu(h[0], h[1], h[2]))

    # ---- not a graded config: the reference's exact int8 matmul (benchmarks/bench_matmul.py:100-131) ----
    def int8_matmul_wl(m, n, k):
        def make(i):
            g = gen(i)
            return (torch.randint(-128, 128, (m, k), device="cuda", dtype=torch.int8, generator=g),
                    torch.randint(-128, 128, (k, n), device="cuda", dtype=torch.int8, generator=g),
                    torch.empty(m, n, device="cuda", dtype=torch.int32))

        return dict(name=f"matmul_int8_{m}x{n}x{k}", kernel="matmul_int", jit=ops.int8_matmul_kernel, unit="TOP/s",
                    bound="tensor", peak_scale=2.0, dtype="s8", work=2 * m * n * k, set_bytes=m * k + k * n + 4 * m * n, make=make,
                    run=lambda s: ops.int_matmul(s[0], s[1], s[2]))

    # ---- config 4: attention bf16 [8, 32, 4096, 128] ----
    def attention_wl(causal):
        z, h, s_, d = 8, 32, 4096, 128

        def make(i):
            g = gen(i)
            q, k, v = (torch.randn(z, h, s_, d, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
            return q, k, v, torch.empty_like(q), torch.empty(z, h, s_, device="cuda")

        flops = 4 * z * h * s_ * s_ * d // (2 if causal else 1)
        zh = 2  # batches of the host (end-to-end) leg: a quarter of the workload, to bound the bench's run time

        def host():
            r = np.random.default_rng(0)
            return tuple(_bf16_host((zh, h, s_, d), r) for _ in range(3))

        return dict(name=f"attention_bf16_8x32x4096x128_{'causal' if causal else 'full'}", kernel="attention",
                    jit=ops.attention_kernel,
                    unit="TFLOP/s", bound="tensor", dtype="bf16", work=flops, set_bytes=4 * z * h * s_ * d * 2,
                    make=make, run=lambda s: ops.attention(s[0], s[1], s[2], causal, None, s[3]),
                    host=host, run_host=lambda hh: ops.attention(hh[0], hh[1], hh[2], causal), host_units=flops * zh // z)

    # ---- config 5: histogram / cumsum ----
    def hist_wl(kind):
        n = int((1 << 30) * scale)
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

        return dict(name=f"histogram_i32_2p30_{kind}", kernel="histogram", jit=ops.histogram_kernel, unit="GB/s", bound="hbm", dtype="i32",
                    work=n * 4, set_bytes=n * 4, make=make, run=run, sets=1,
                    host=lambda: (np.random.default_rng(0).integers(0, bins, n // 16).astype(np.int32),),
                    run_host=lambda h: ops.histogram(h[0], bins, 0.0, float(bins)), host_units=(n // 16) * 4,
                    cpu=lambda h: O.histogram(h[0], bins, 0.0, float(bins)), cpu_units=(n // 16) * 4)

    def cumsum_wl(kind):
        from enceladus_b200 import dist as edist

        n = int((1 << 30) * scale) if kind == "i32" else int((1 << 28) * scale)

        def make(i):
            g = gen(i)
            if kind == "i32":
                x = torch.randint(0, 16, (n,), device="cuda", dtype=torch.int32, generator=g)
            else:
                x = torch.randn(n, device="cuda", generator=g)
            return x, torch.empty_like(x), torch.zeros(1, device="cuda", dtype=x.dtype)

        def run(s):
            if WORLD > 1:  # local total -> all-gather -> seeded local scan (reads the shard twice)
                edist.sharded_cumsum(s[0], edist.cuda_total, lambda x, seed: _scan_into(x, s[1], seed))
            else:
                ops.cumsum_kernel[(1,)](s[1], s[0], 1, n, n, n, REVERSE=False, BLOCK_M=1, BLOCK_N=1 << 30)

        def _scan_into(x, out, seed):
            from enceladus_b200.runtime import interop

            N.call("enc_cumsum", x.data_ptr(), out.data_ptr(), 1, n, n, n, 0, interop.dtype_code(x),
                   seed.data_ptr(), -1, interop.current_stream())
            return out

        nh = n // 16
        return dict(name=f"cumsum_{kind}_{'2p30' if kind == 'i32' else '2p28'}", kernel="cumsum", jit=ops.cumsum_kernel, unit="GB/s",
                    bound="hbm", dtype=kind, work=2 * n * 4, set_bytes=2 * n * 4, make=make, run=run, sets=1,
                    host=lambda: ((np.random.default_rng(0).integers(0, 16, nh).astype(np.int32),) if kind == "i32"
                                  else (np.random.default_rng(0).standard_normal(nh).astype(np.float32),)),
                    run_host=lambda h: ops.cumsum(h[0]), host_units=2 * nh * 4,
                    cpu=lambda h: O.cumsum(h[0]), cpu_units=2 * nh * 4)

    W["softmax"] = softmax_wl
    W["softmax_4096x4096"] = lambda: softmax_wl(4096)  # the reference's own benchmark shape (benchmarks/bench_softmax.py)
    W["layernorm"] = lambda: norm_wl("layernorm")
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


USE_GRAPH = True
RANK = int(os.environ.get("RANK", "0"))
LOCAL_RANK = int(os.environ.get("LOCAL_RANK", "0"))
WORLD = int(os.environ.get("WORLD_SIZE", "1"))


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


def bench_workload(wl: dict, steps: int, warmup: int, pk: dict, pk_kind: str, sampler, e2e: bool, cpu: bool,
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
    m1 = sampler.mark() if sampler else 0
    achieved = wl["work"] / (ms * 1e-3) / (1e9 if wl["unit"] == "GB/s" else 1e12)
    peak = pk["hbm_gbs"] if wl["bound"] == "hbm" else pk["bf16_tflops"] * wl.get("peak_scale", 1.0)
    if "peak_scale" in wl:  # no int8 GEMM was measured on this pool: the 8-bit rate of the tensor cores is twice the 16-bit one
        pk_kind = f"{wl['peak_scale']:g} x {pk_kind} bf16"
    row = {
        "name": wl["name"], "value": achieved * WORLD, "unit": wl["unit"], "ms_per_step": ms, "steps": steps,
        "warmup": warmup, "dtype": wl["dtype"], "buffer_sets": nsets, "cuda_graph": graph,
        "roofline": {"bound": wl["bound"], "achieved": achieved, "peak": peak, "unit": wl["unit"],
                     "frac": achieved / peak, "peak_source": pk_kind, "traffic": NCU_TRAFFIC.get(wl["name"])},
    }
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
        row["e2e"] = {"value": units * WORLD / (dev_ms * 1e-3) / (1e9 if wl["unit"] == "GB/s" else 1e12), "unit": wl["unit"],
                      "h2d_bytes_per_step": int(last.get("h2d_bytes", 0)),
                      "d2h_bytes_per_step": int(sum(r.nbytes for r in res)), "ms_per_step": dev_ms,
                      "workload_fraction": units / wl["work"]}
        if cpu and RANK == 0:
            row["cpu_baseline"] = cpu_baseline(wl, h, threads=1)
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
        value = work / (ms * 1e-3) / (1e9 if unit == "GB/s" else 1e12)
        peak = pk["hbm_gbs"] if bound == "hbm" else pk["bf16_tflops"] * (2.0 if unit == "TOP/s" else 1.0)
        rows.append({"name": name, "value": value, "unit": unit, "ms_per_step": ms, "steps": steps, "frac_of_peak": value / peak,
                     "published_m4pro": published, "vs_published": value / published if published else None})
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


def cpu_baseline(wl: dict, h, threads: int, budget_s: float = 20.0) -> dict:
    """Times the NumPy restatement of the reference on a bounded sample of the workload's host input."""
    units = wl.get("cpu_units", wl["work"])
    rows = wl.get("cpu_rows")
    sample = "whole host workload"
    if rows:  # row-wise workloads: time a slice of rows sized for the budget
        probe = 256
        t0 = time.perf_counter()
        wl["cpu"](h, probe)
        per_row = (time.perf_counter() - t0) / probe
        take = int(max(probe, min(rows, budget_s / max(per_row, 1e-9) * max(threads, 1))))
        units = wl["row_bytes"] * take
        sample = f"{take} of {rows} rows"
        if threads > 1:
            chunks = np.array_split(np.arange(take), threads)
            t0 = time.perf_counter()
            with ThreadPoolExecutor(threads) as pool:
                list(pool.map(lambda c: wl["cpu"]((h[0][c[0] : c[-1] + 1], *h[1:])), [c for c in chunks if len(c)]))
            dt = time.perf_counter() - t0
        else:
            t0 = time.perf_counter()
            wl["cpu"](h, take)
            dt = time.perf_counter() - t0
    else:
        t0 = time.perf_counter()
        wl["cpu"](h)
        dt = time.perf_counter() - t0
        if "host_units" in wl and wl["host_units"] != wl["work"]:
            sample = f"{wl['host_units'] / wl['work']:.4f} of the workload"
    scale = 1e9 if wl["unit"] == "GB/s" else 1e12
    return {"value": units / dt / scale, "unit": wl["unit"], "cores": threads, "kind": "port",
            "sample": f"{sample}; NumPy restatement of the reference interpreter, {dt:.2f} s"}


def reference_arm(args) -> None:
    """`--impl reference`: the CPU restatement of the reference on all host threads, rank 0 only."""
    if RANK != 0:
        return
    import ml_dtypes  # noqa: F401

    from oracle import enceladus_oracle as O

    cores = len(os.sched_getaffinity(0))
    m, n = 16384, 4096
    r = np.random.default_rng(0)
    h = (_bf16_host((m, n), r), _bf16_host(n, r, 0.1, 1.0), _bf16_host(n, r, 0.1))
    wl = dict(name="layernorm_bf16_16384x4096", unit="GB/s", work=2 * m * n * 2, cpu_rows=m, row_bytes=2 * n * 2,
              cpu=lambda hh, rows=None: O.layernorm(hh[0][:rows], hh[1], hh[2], 1e-5))
    samples = []
    info = None
    for i in range(args.warmup + args.steps):
        info = cpu_baseline(wl, h, threads=cores, budget_s=1.0)
        if i >= args.warmup:
            samples.append(info["value"])
    value = float(np.mean(samples))
    rows_bytes = 2 * m * n * 2
    line = {"impl": "reference", "metric": "layernorm_bf16_16384x4096 algorithmic HBM GB/s (read+write)",
            "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": rows_bytes / (value * 1e9) * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "layernorm_bf16_16384x4096"},
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": info["sample"]},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="layernorm")
    ap.add_argument("--kernels", default="all", help="per_kernel rows: all, none, or a comma list")
    ap.add_argument("--kernel-steps", type=int, default=10)
    ap.add_argument("--scale", type=float, default=1.0, help="shrinks the 2^30 / 2^28 element workloads")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch the timed steps eagerly instead of as one CUDA graph")
    ap.add_argument("--cpu-baseline-all", action="store_true")
    ap.add_argument("--no-reference-shapes", action="store_true", help="skip the rows at the reference's own benchmark shapes")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    global USE_GRAPH
    USE_GRAPH = not args.no_graph

    if args.impl == "reference":
        reference_arm(args)
        return

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
    W = workloads(args.scale)
    if args.workload not in W:
        raise SystemExit(f"unknown workload {args.workload!r}; choose from {sorted(W)}")
    sampler = ClockSampler(visible_gpu_index(LOCAL_RANK)) if RANK == 0 else None
    time.sleep(0.3)

    head = bench_workload(W[args.workload](), args.steps, args.warmup, pk, pk_kind, sampler,
                          e2e=not args.no_e2e, cpu=True)
    rows = []
    launches = args.steps
    if args.kernels != "none":
        names = [k for k in W if k != args.workload] if args.kernels == "all" else args.kernels.split(",")
        for k in names:
            try:
                rows.append(bench_workload(W[k](), args.kernel_steps, 3, pk, pk_kind, sampler,
                                           e2e=not args.no_e2e, cpu=args.cpu_baseline_all, min_region_ms=1.0))
                launches += rows[-1]["steps"]
            except Exception as e:  # noqa: BLE001 - one failing workload must not hide the others
                rows.append({"name": k, "error": f"{type(e).__name__}: {e}"})
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
    line = {
        "metric": f"{head['name']} algorithmic {'HBM GB/s (read+write)' if head['unit'] == 'GB/s' else 'TFLOP/s'}",
        "value": head["value"], "unit": head["unit"], "n_gpus": WORLD, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": head["dtype"], "data": "synthetic",
        "config": {"workload": head["name"], "l2": f"rotating {head['buffer_sets']} buffer sets (> 4x L2 in total)",
                   "sharding": "same per-GPU workload on every rank, no data-path collective",
                   "timed_region": "K launches captured in one CUDA graph" if head.get("cuda_graph") else "K eager launches"},
        "roofline": head["roofline"], "clocks": head.get("clocks"), "gpu_launches": launches,
        "e2e": head.get("e2e"), "cpu_baseline": head.get("cpu_baseline"), "per_kernel": rows,
        "reference_shapes": ref_rows,
    }
    print(json.dumps(line))


if __name__ == "__main__":
    main()
