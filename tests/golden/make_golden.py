"""Generates the golden vectors in this directory by running the reference itself.

The reference (kashifulhaque/enceladus) is a Python project whose CPU interpreter
(`ENCELADUS_INTERPRET=1`) needs only NumPy and ml_dtypes.  Its package imports the Metal extension
`enceladus._C` at import time, so a placeholder module carrying `MetalError` and empty handle classes
is registered first; the interpreter path never touches the device.

Usage (on a machine that has the reference checkout):

    python tests/golden/make_golden.py --reference /path/to/enceladus [--out tests/golden]

Every case uses the shapes, dtypes and seeds of the reference's own tests
(tests/test_interpreter.py:44-113, tests/test_attention.py:20-49,
tests/test_atomics_scans.py:200-227) plus small cases of the benchmark configurations.  Inputs and
interpreter outputs are written to `<kernel>.npz`; bfloat16 arrays are stored as uint16 bit patterns
with a `__bf16` suffix on the key.  Large outputs are stored as a SHA-256 of their bytes.
"""

from __future__ import annotations

import argparse
import hashlib
import importlib
import os
import sys
import types
from pathlib import Path

import ml_dtypes
import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from enceladus_b200.workloads import zipf_clipped  # noqa: E402

BF16 = np.dtype(ml_dtypes.bfloat16)
F16, F32 = np.dtype(np.float16), np.dtype(np.float32)
NAMES = {F32: "f32", F16: "f16", BF16: "bf16"}


def import_reference(root: str):
    os.environ["ENCELADUS_INTERPRET"] = "1"
    os.environ["ENCELADUS_VERIFY"] = "0"
    stub = types.ModuleType("enceladus._C")
    stub.MetalError = type("MetalError", (RuntimeError,), {})
    for n in ("Buffer", "Pipeline", "Queue", "Stream", "LaunchPlan", "Device", "Library"):
        setattr(stub, n, type(n, (), {}))
    sys.modules["enceladus._C"] = stub
    sys.path.insert(0, os.path.join(root, "src"))
    sys.path.insert(0, os.path.join(root, "examples"))
    import enceladus  # noqa: F401

    return lambda name: importlib.import_module(name)


def randn(rng, shape, dtype):
    return rng.standard_normal(shape).astype(np.float32).astype(dtype)


class Bag(dict):
    def put(self, key: str, arr):
        arr = np.asarray(arr)
        if arr.dtype == BF16:
            self[key + "__bf16"] = arr.view(np.uint16)
        else:
            self[key] = arr


def sha(arr) -> np.ndarray:
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(arr).tobytes()).digest(), np.uint8)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("ENCELADUS_REFERENCE"), required="ENCELADUS_REFERENCE" not in os.environ,
                    help="checkout of kashifulhaque/enceladus (or set ENCELADUS_REFERENCE)")
    ap.add_argument("--out", default=str(Path(__file__).parent))
    a = ap.parse_args()
    ex = import_reference(a.reference)
    import enceladus
    import enceladus.language as tl

    out = Path(a.out)

    # ---- softmax: tests/test_interpreter.py:44-49 and benchmark config 1 ----
    g = Bag()
    m = ex("02_softmax")
    rng = np.random.default_rng(1234)
    for dt in (F32, F16):
        for shape in ((4, 128), (37, 1000), (3, 20)):
            k = f"{NAMES[dt]}_{shape[0]}x{shape[1]}"
            x = randn(rng, shape, dt) * dt.type(4)
            g.put(k + "_x", x)
            g.put(k + "_y", m.softmax(x))
    x = np.random.default_rng(0).standard_normal((4096, 1024)).astype(np.float32) * 4
    y = m.softmax(x)
    g.put("config1_sha256", sha(y))
    g.put("config1_rows0_8", y[:8])
    np.savez_compressed(out / "softmax.npz", **g)

    # ---- layernorm: tests/test_interpreter.py:52-59, plus bf16 rows of the config-2 width ----
    g = Bag()
    m = ex("03_layernorm")
    for dt in (F32, F16):
        for shape, block in (((8, 256), 256), ((5, 1000), 256)):
            k = f"{NAMES[dt]}_{shape[0]}x{shape[1]}_b{block}"
            x = randn(rng, shape, dt) * dt.type(2) + dt.type(1)
            w, b = randn(rng, shape[1], dt), randn(rng, shape[1], dt)
            y, mean, rstd = m.layernorm(x, w, b, block=block)
            for n, v in (("x", x), ("w", w), ("b", b), ("y", y), ("mean", mean), ("rstd", rstd)):
                g.put(f"{k}_{n}", v)
    r2 = np.random.default_rng(2)
    x = r2.standard_normal((12, 4096)).astype(np.float32).astype(BF16)
    w = (1 + 0.1 * r2.standard_normal(4096)).astype(np.float32).astype(BF16)
    b = (0.1 * r2.standard_normal(4096)).astype(np.float32).astype(BF16)
    y, mean, rstd = m.layernorm(x, w, b, eps=1e-5)
    for n, v in (("x", x), ("w", w), ("b", b), ("y", y), ("mean", mean), ("rstd", rstd)):
        g.put(f"bf16_12x4096_b1024_{n}", v)
    np.savez_compressed(out / "layernorm.npz", **g)

    # ---- rmsnorm: tests/test_interpreter.py:108-113 ----
    g = Bag()
    m = ex("06_rmsnorm")
    for dt in (F32, F16):
        for shape in ((4, 128), (9, 1000)):
            k = f"{NAMES[dt]}_{shape[0]}x{shape[1]}"
            x, w = randn(rng, shape, dt), randn(rng, shape[1], dt)
            g.put(k + "_x", x), g.put(k + "_w", w), g.put(k + "_y", m.rmsnorm(x, w))
    x = r2.standard_normal((12, 4096)).astype(np.float32).astype(BF16)
    w = (1 + 0.1 * r2.standard_normal(4096)).astype(np.float32).astype(BF16)
    g.put("bf16_12x4096_x", x), g.put("bf16_12x4096_w", w)
    g.put("bf16_12x4096_y", m.rmsnorm(x, w, eps=1e-6))
    np.savez_compressed(out / "rmsnorm.npz", **g)

    # ---- fused GELU: tests/test_interpreter.py:100-105; tanh form through a DSL kernel ----
    g = Bag()
    m = ex("05_fused_gelu")
    for dt in (F32, F16, BF16):
        for shape in ((4, 256), (7, 300)):
            k = f"{NAMES[dt]}_{shape[0]}x{shape[1]}"
            x, bias = randn(rng, shape, dt), randn(rng, shape[1], dt)
            g.put(k + "_x", x), g.put(k + "_bias", bias)
            g.put(k + "_y", m.fused_gelu(x, bias, 0.75))

    @enceladus.jit
    def tanh_gelu_kernel(x_ptr, out_ptr, n, BLOCK: tl.constexpr):
        offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
        mask = offs < n
        x = tl.load(x_ptr + offs, mask=mask).to(tl.float32)
        inner = 0.7978845608028654 * (x + 0.044715 * x * x * x)
        tl.store(out_ptr + offs, 0.5 * x * (1.0 + tl.tanh(inner)), mask=mask)

    x = (np.random.default_rng(3).standard_normal(20_003) * 2).astype(np.float32)
    y = np.empty_like(x)
    tanh_gelu_kernel[(enceladus.cdiv(x.size, 1024),)](x, y, x.size, BLOCK=1024)
    g.put("tanh_f32_x", x), g.put("tanh_f32_y", y)
    np.savez_compressed(out / "gelu.npz", **g)

    # ---- matmul: tests/test_interpreter.py:65-97 ----
    g = Bag()
    m = ex("07_matmul_fused")
    for dt in (F32, F16):
        aa, bb = randn(rng, (200, 96), dt), randn(rng, (96, 130), dt)
        bias = randn(rng, 130, dt)
        k = f"fused_{NAMES[dt]}_200x96x130"
        g.put(k + "_a", aa), g.put(k + "_b", bb), g.put(k + "_bias", bias)
        g.put(k + "_c", m.matmul_bias_gelu(aa, bb, bias))
    r3 = np.random.default_rng(7)
    aa = (r3.uniform(-1, 1, (256, 512)) / np.sqrt(512)).astype(F16)
    bb = (r3.uniform(-1, 1, (512, 384)) / np.sqrt(512)).astype(F16)
    bias = (0.1 * r3.standard_normal(384)).astype(F16)
    g.put("fused_f16_256x512x384_a", aa), g.put("fused_f16_256x512x384_b", bb)
    g.put("fused_f16_256x512x384_bias", bias)
    g.put("fused_f16_256x512x384_c", m.matmul_bias_gelu(aa, bb, bias, bm=64, bn=64, bk=64))
    m4 = ex("04_matmul")
    for dt in (F32, F16, BF16):
        aa, bb = randn(rng, (100, 70), dt), randn(rng, (70, 90), dt)
        k = f"plain_{NAMES[dt]}_100x70x90"
        g.put(k + "_a", aa), g.put(k + "_b", bb), g.put(k + "_c", m4.matmul_desc(aa, bb))
    np.savez_compressed(out / "matmul.npz", **g)

    # ---- integer matmul: tests/test_interpreter.py:808-835 (shapes, dtypes, full-range values) ----
    # The kernel below is written for this script (pointer loads with edge masks, one tl.dot per K block into
    # an int32 accumulator) and executed by the reference interpreter.
    @enceladus.jit
    def int_dot_kernel(a_ptr, b_ptr, c_ptr, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
        rm = tl.program_id(1) * BM + tl.arange(0, BM)
        rn = tl.program_id(0) * BN + tl.arange(0, BN)
        acc = tl.zeros((BM, BN), dtype=tl.int32)
        for k0 in range(0, K, BK):
            rk = k0 + tl.arange(0, BK)
            at = tl.load(a_ptr + rm[:, None] * K + rk[None, :], mask=(rm[:, None] < M) & (rk[None, :] < K), other=0)
            bt = tl.load(b_ptr + rk[:, None] * N + rn[None, :], mask=(rk[:, None] < K) & (rn[None, :] < N), other=0)
            acc = tl.dot(at, bt, acc)
        tl.store(c_ptr + rm[:, None] * N + rn[None, :], acc, mask=(rm[:, None] < M) & (rn[None, :] < N))

    g = Bag()
    r5 = np.random.default_rng(11)
    for dt in (np.int8, np.uint8, np.int16, np.int32):
        for (mm, kk_, nn) in ((64, 64, 64), (50, 100, 33)):
            info = np.iinfo(dt)
            aa = r5.integers(info.min, info.max, (mm, kk_), dt, endpoint=True)
            bb = r5.integers(info.min, info.max, (kk_, nn), dt, endpoint=True)
            cc = np.zeros((mm, nn), np.int32)
            int_dot_kernel[(enceladus.cdiv(nn, 32), enceladus.cdiv(mm, 32))](aa, bb, cc, mm, nn, kk_, BM=32, BN=32, BK=32)
            key = f"{np.dtype(dt).name}_{mm}x{kk_}x{nn}"
            g.put(key + "_a", aa), g.put(key + "_b", bb), g.put(key + "_c", cc)
    # every sum exceeds 2^24 and is odd: float32 accumulation would round it (test_interpreter.py:822-835)
    for dt, kk_ in ((np.int8, 2048), (np.uint8, 512)):
        ext = np.iinfo(dt).min if dt == np.int8 else np.iinfo(dt).max
        aa, bb = np.full((8, kk_), ext, dt), np.full((kk_, 8), ext, dt)
        aa[:, 0] = 1
        cc = np.zeros((8, 8), np.int32)
        int_dot_kernel[(1, 1)](aa, bb, cc, 8, 8, kk_, BM=8, BN=8, BK=32)
        key = f"exact_{np.dtype(dt).name}_{kk_}"
        g.put(key + "_a", aa), g.put(key + "_b", bb), g.put(key + "_c", cc)
    np.savez_compressed(out / "int_matmul.npz", **g)

    # ---- attention: tests/test_attention.py:20-49 (inputs are regenerated from the seed) ----
    g = Bag()
    m = ex("08_flash_attention")
    cases = [(F16, 64, 64, False, (32, 32, 4)), (F16, 64, 64, True, (32, 32, 4)),
             (F16, 100, 64, False, (32, 32, 4)), (F16, 100, 64, True, (32, 32, 4)),
             (F16, 100, 128, False, (64, 32, 8)), (F16, 100, 128, True, (32, 16, 4)),
             (F16, 100, 64, True, (64, 16, 4)), (F16, 37, 32, False, (16, 32, 1)),
             (F32, 100, 128, True, (32, 32, 4)), (BF16, 100, 64, False, (32, 16, 4)),
             (BF16, 200, 128, True, (64, 32, 8)), (BF16, 200, 128, False, (64, 32, 8))]
    for i, (dt, n, d, causal, (bm, bn, nw)) in enumerate(cases):
        r = np.random.default_rng(n + d)
        q, kk, v = (r.standard_normal((2, 2, n, d)).astype(np.float32).astype(dt) for _ in range(3))
        o = m.attention(q, kk, v, causal, 0.3 if causal else None, block_m=bm, block_n=bn,
                        num_warps=nw)
        code = {"f32": 0, "f16": 1, "bf16": 2}[NAMES[dt]]
        g.put(f"case{i}_meta", np.array([n, d, int(causal), bm, bn, code], np.int64))
        g.put(f"case{i}_o", o)
    np.savez_compressed(out / "attention.npz", **g)

    # ---- histogram: tests/test_atomics_scans.py:200-205, plus int32 inputs of config 5 ----
    g = Bag()
    m = ex("09_histogram")
    x = np.random.default_rng(5).standard_normal(100_003).astype(np.float32)
    g.put("f32_100003_48bins", m.histogram(x, 48, -3.0, 3.0))
    x = np.random.default_rng(0).integers(0, 256, 1 << 18).astype(np.int32)
    g.put("i32_uniform256_2p18", m.histogram(x, 256, 0.0, 256.0))
    g.put("i32_zipf4096_2p16", m.histogram(zipf_clipped(np.random.default_rng(1), 1 << 16, 1.1, 4096),
                                           4096, 0.0, 4096.0))
    np.savez_compressed(out / "histogram.npz", **g)

    # ---- cumsum: tests/test_atomics_scans.py:214-227, plus an int32 row that wraps ----
    g = Bag()
    m = ex("10_cumsum")
    for dt in (F32, F16, BF16, np.dtype(np.int8), np.dtype(np.int64), np.dtype(np.int32)):
        for shape in ((5, 1000), (64, 32), (3, 7)):
            r = np.random.default_rng(shape[1])
            if dt.kind in "iu":
                x = r.integers(-100, 100, shape).astype(dt)
            else:
                x = (r.standard_normal(shape) * 4).astype(np.float32).astype(dt)
            for rev in (False, True):
                name = NAMES.get(dt, dt.name)
                g.put(f"{name}_{shape[0]}x{shape[1]}_rev{int(rev)}", m.cumsum(x, reverse=rev))
    x = np.random.default_rng(9).integers(0, 1 << 20, (2, 65536)).astype(np.int32)
    y = m.cumsum(x)
    g.put("i32_wrap_2x65536_sha256", sha(y))
    g.put("i32_wrap_2x65536_tail", y[:, -16:])
    np.savez_compressed(out / "cumsum.npz", **g)
    print("golden vectors written to", out)


if __name__ == "__main__":
    main()
