"""CPU restatement (NumPy) of the arithmetic the Enceladus interpreter applies to the kernel set.

TEST INFRASTRUCTURE ONLY.  This module is the *checker*: the tests, the smoke check and the
benchmark's CPU-baseline leg may call it; no product code path imports it, and the CUDA path never
falls back to it.

Every function follows the reference kernel body line by line, using the NumPy call the reference
interpreter makes for each `tl.*` builtin, so that results agree with the interpreter bit for bit
wherever NumPy's own evaluation order allows (same padded tile widths, same per-op float32
rounding, same pairwise `np.sum`).  The pins are the golden vectors under `tests/golden/`, which were
produced by the reference interpreter itself (`ENCELADUS_INTERPRET=1`) with
`tests/golden/make_golden.py`.

Interpreter rules restated here (paths are inside the reference project):
  * each float op computes in float32 and rounds after every op   src/enceladus/interpreter/interp.py:635-690
  * Python literals become float32 constants                      src/enceladus/interpreter/interp.py:510-548
  * float scalar kernel arguments are float32                     src/enceladus/runtime/jit.py:124-125
  * tl.sum = np.sum(dtype=float32), tl.max = np.fmax.reduce       src/enceladus/language/ops.py:945-975
  * tl.dot = float32 `@` of the K-block plus accumulator          src/enceladus/language/ops.py:1222-1240
  * tl.cumsum = np.cumsum in int32 / float32                      src/enceladus/language/ops.py:2047-2060
  * tl.erf = math.erf in float64, then cast                       src/enceladus/interpreter/interp.py:608-609
  * tl.rsqrt = 1/np.sqrt                                          src/enceladus/interpreter/interp.py:663
  * float -> int32 truncates and saturates                        src/enceladus/interpreter/interp.py:573-597
  * stores round to the pointee dtype (RNE; bf16 via ml_dtypes)   src/enceladus/language/ops.py:339-361
  * descriptor loads zero-fill, descriptor stores skip OOB        src/enceladus/language/ops.py:495-514
"""

from __future__ import annotations

import math

import numpy as np

try:  # bfloat16 for NumPy; the reference depends on it too (pyproject.toml:13)
    import ml_dtypes

    bfloat16 = np.dtype(ml_dtypes.bfloat16)
except ImportError:  # pragma: no cover
    ml_dtypes = None
    bfloat16 = None

try:
    from scipy.special import erf as _erf64
except ImportError:  # pragma: no cover
    _erf64 = np.vectorize(math.erf, otypes=[np.float64])

F32 = np.float32
_SQRT1_2 = F32(0.7071067811865476)  # literal of examples/05_fused_gelu.py:25, rounded to float32
_LOG2E = F32(1.4426950408889634)  # literal of examples/08_flash_attention.py:49


def next_power_of_2(n: int) -> int:
    """src/enceladus/runtime/jit.py:69-71."""
    return 1 if n <= 1 else 1 << (int(n) - 1).bit_length()


def _f32(x: np.ndarray) -> np.ndarray:
    """`.to(tl.float32)` of a loaded tile (exact for fp16/bf16)."""
    return np.asarray(x).astype(F32)


def _store(y: np.ndarray, dtype) -> np.ndarray:
    """`tl.store`: float32 value rounded to the pointee dtype."""
    return np.asarray(y).astype(dtype)


def _erf(x: np.ndarray) -> np.ndarray:
    return _erf64(x.astype(np.float64)).astype(x.dtype)


def _pad_cols(x: np.ndarray, width: int, fill) -> np.ndarray:
    """A masked load of `width` lanes over rows of `x`: lanes past the row read `fill`."""
    m, n = x.shape
    if n == width:
        return x
    out = np.full((m, width), fill, dtype=x.dtype)
    out[:, :n] = x
    return out


# ---------------------------------------------------------------------------------------------
# Row softmax — examples/02_softmax.py:15-38
# ---------------------------------------------------------------------------------------------
def softmax(x: np.ndarray) -> np.ndarray:
    m, n = x.shape
    block = next_power_of_2(n)
    t = _pad_cols(_f32(x), block, F32(-np.inf))  # :19-20 masked load, other=-inf, .to(f32)
    t = t - np.fmax.reduce(t, axis=1, keepdims=True)  # :21
    num = np.exp(t)  # :22
    den = np.sum(num, axis=1, keepdims=True, dtype=F32)  # :23 tl.sum over BLOCK lanes
    return _store((num / den)[:, :n], x.dtype)


# ---------------------------------------------------------------------------------------------
# LayerNorm — examples/03_layernorm.py:15-57
# ---------------------------------------------------------------------------------------------
def layernorm(x, w, b, eps: float = 1e-5, block: int | None = None):
    """Returns (y, mean, rstd); statistics float32, y in x's dtype."""
    m, n = x.shape
    block = block or min(1024, next_power_of_2(n))  # :54
    nchunks = -(-n // block)
    width = nchunks * block
    xf = _pad_cols(_f32(x), width, F32(0.0)).reshape(m, nchunks, block)
    valid = (np.arange(width) < n).reshape(1, nchunks, block)
    n_i = F32(n)  # fp32 / int32 divides in fp32 (compiler/semantic.py:147-148)
    acc = np.zeros((m, block), F32)
    for c in range(nchunks):  # :21-23 per-lane partial sums, chunk by chunk
        acc = acc + xf[:, c, :]
    mean = np.sum(acc, axis=1, dtype=F32) / n_i  # :24
    acc = np.zeros((m, block), F32)
    for c in range(nchunks):  # :26-30
        d = np.where(valid[:, c, :], xf[:, c, :] - mean[:, None], F32(0.0))
        acc = acc + d * d
    var = np.sum(acc, axis=1, dtype=F32) / n_i  # :31
    rstd = F32(1.0) / np.sqrt(var + F32(eps))  # :32
    wf, bf = _f32(w)[None, :], _f32(b)[None, :]
    xr = xf.reshape(m, width)[:, :n]
    y = (xr - mean[:, None]) * rstd[:, None] * wf + bf  # :42, left to right, one rounding per op
    return _store(y, x.dtype), mean.astype(F32), rstd.astype(F32)


# ---------------------------------------------------------------------------------------------
# RMSNorm — examples/06_rmsnorm.py:15-37
# ---------------------------------------------------------------------------------------------
def rmsnorm(x, w, eps: float = 1e-6):
    m, n = x.shape
    block = next_power_of_2(n)
    t = _pad_cols(_f32(x), block, F32(0.0))  # :21
    ms = np.sum(t * t, axis=1, dtype=F32) / F32(n)
    rstd = F32(1.0) / np.sqrt(ms + F32(eps))  # :22 tl.rsqrt = 1/np.sqrt
    y = t[:, :n] * rstd[:, None] * _f32(w)[None, :]  # :24
    return _store(y, x.dtype)


# ---------------------------------------------------------------------------------------------
# Fused GELU — examples/05_fused_gelu.py:17-33 (erf form) and the tanh form expressed with tl.tanh
# ---------------------------------------------------------------------------------------------
def fused_gelu(x, bias, scale: float) -> np.ndarray:
    """`gelu_erf(x*scale + bias[col])` for a contiguous 2-D x and a per-column bias."""
    n_cols = x.shape[-1]
    flat = _f32(x).reshape(-1)
    offs = np.arange(flat.size, dtype=np.int64)
    bb = _f32(bias)[offs % n_cols]  # :22
    y = flat * F32(scale) + bb  # :23 two roundings
    out = F32(0.5) * y * (F32(1.0) + _erf(y * _SQRT1_2))  # :25
    return _store(out.reshape(x.shape), x.dtype)


def gelu_erf(x) -> np.ndarray:
    """Elementwise erf-GELU with no scale and no bias (same expression as fused_gelu)."""
    y = _f32(x)
    return _store(F32(0.5) * y * (F32(1.0) + _erf(y * _SQRT1_2)), x.dtype)


def gelu_tanh(x) -> np.ndarray:
    """`0.5*x*(1 + tanh(0.7978845608*(x + 0.044715*x*x*x)))`, each op rounded to float32.

    The reference ships no tanh kernel; this is the expression a DSL kernel built from `tl.tanh`
    (= np.tanh, src/enceladus/interpreter/interp.py:666) evaluates, left to right:
        inner = 0.7978845608028654 * (x + 0.044715 * x * x * x)
        out   = 0.5 * x * (1.0 + tl.tanh(inner))
    """
    y = _f32(x)
    inner = F32(0.7978845608028654) * (y + F32(0.044715) * y * y * y)
    return _store(F32(0.5) * y * (F32(1.0) + np.tanh(inner)), x.dtype)


# ---------------------------------------------------------------------------------------------
# Matmul (+bias +GELU) — examples/07_matmul_fused.py:17-48, examples/04_matmul.py:21-63
# ---------------------------------------------------------------------------------------------
def matmul(a, b, bk: int = 32, out_dtype=None) -> np.ndarray:
    """float32 accumulation over K in blocks of `bk`, in order (one `tl.dot` per block)."""
    k = a.shape[1]
    af, bf = _f32(a), _f32(b)
    acc = np.zeros((a.shape[0], b.shape[1]), F32)
    for k0 in range(0, k, bk):
        acc = af[:, k0 : k0 + bk] @ bf[k0 : k0 + bk, :] + acc  # language/ops.py:1239
    return _store(acc, out_dtype or a.dtype)


def matmul_bias_gelu(a, b, bias, bk: int = 32) -> np.ndarray:
    acc = matmul(a, b, bk, out_dtype=F32)
    y = acc + _f32(bias)[None, :]  # :29
    y = F32(0.5) * y * (F32(1.0) + _erf(y * _SQRT1_2))  # :30
    return _store(y, a.dtype)


def int_matmul(a, b) -> np.ndarray:
    """Integer `tl.dot`: int32 accumulation, exact, products and sums wrap modulo 2^32
    (src/enceladus/language/ops.py:1255-1259; the reference's own check is
    tests/test_interpreter.py:804-805: the int64 product cast to int32)."""
    return (a.astype(np.int64) @ b.astype(np.int64)).astype(np.int32)


# ---------------------------------------------------------------------------------------------
# Flash-attention forward — examples/08_flash_attention.py:30-70
# ---------------------------------------------------------------------------------------------
def attention(q, k, v, causal: bool = False, sm_scale: float | None = None, block_m: int = 32,
              block_n: int = 32, return_lse: bool = False):
    """Online-softmax attention over (batch, heads, seq, dim); all heads advance together.

    The logsumexp output is an addition of this build (the reference kernel stores only O): it is
    `ln2 * (m_i + log2(l_i))` from the kernel's own running statistics, in float32, i.e. what one
    extra `tl.store` of `(m_i + tl.log2(l_i)) * 0.6931471805599453` would write.
    """
    z, h, n, d = q.shape
    dt = q.dtype
    scale = 1.0 / math.sqrt(d) if sm_scale is None else sm_scale
    qk_scale = F32(scale) * _LOG2E  # :49 (f32 scalar arg times f32 constant)
    qf, kf, vf = (_f32(t).reshape(z * h, n, d) for t in (q, k, v))
    out = np.empty((z * h, n, d), dt)
    lse = np.empty((z * h, n), F32)
    for m0 in range(0, n, block_m):
        rows = np.arange(m0, m0 + block_m)
        qt = np.zeros((z * h, block_m, d), F32)  # descriptor load zero-fills rows past N_CTX
        nv = min(block_m, n - m0)
        qt[:, :nv] = qf[:, m0 : m0 + nv]
        m_i = np.full((z * h, block_m), -np.inf, F32)
        l_i = np.zeros((z * h, block_m), F32)
        acc = np.zeros((z * h, block_m, d), F32)
        hi = min(m0 + block_m, n) if causal else n  # :52-54
        for n0 in range(0, hi, block_n):
            cols = np.arange(n0, n0 + block_n)
            kt = np.zeros((z * h, block_n, d), F32)
            vt = np.zeros((z * h, block_n, d), F32)
            cv = min(block_n, n - n0)
            kt[:, :cv] = kf[:, n0 : n0 + cv]
            vt[:, :cv] = vf[:, n0 : n0 + cv]
            qk = np.matmul(qt, kt.transpose(0, 2, 1)) * qk_scale  # :56
            mask = np.broadcast_to(cols[None, :] < n, (block_m, block_n))
            if causal:
                mask = mask & (rows[:, None] >= cols[None, :])
            qk = np.where(mask[None], qk, F32(-np.inf))  # :61
            m_ij = np.fmax(m_i, np.fmax.reduce(qk, axis=2))  # :62
            with np.errstate(invalid="ignore"):
                p = np.exp2(qk - m_ij[:, :, None])  # :63
                alpha = np.exp2(m_i - m_ij)  # :64
            l_i = l_i * alpha + np.sum(p, axis=2, dtype=F32)  # :65
            acc = acc * alpha[:, :, None]  # :66
            acc = np.matmul(p.astype(dt).astype(F32), vt) + acc  # :67 P rounded to input dtype
            m_i = m_ij
        acc = acc / l_i[:, :, None]  # :69
        out[:, m0 : m0 + nv] = acc[:, :nv].astype(dt)
        lse[:, m0 : m0 + nv] = ((m_i + np.log2(l_i)) * F32(0.6931471805599453))[:, :nv]
    out = out.reshape(z, h, n, d)
    return (out, lse.reshape(z, h, n)) if return_lse else out


def attention_lse_f64(q, k, v, causal: bool = False, sm_scale: float | None = None):
    """float64 logsumexp(scale * q k^T) per row, after examples/08_flash_attention.py:130-140."""
    d = q.shape[-1]
    scale = 1.0 / math.sqrt(d) if sm_scale is None else sm_scale
    s = np.einsum("zhmd,zhnd->zhmn", q.astype(np.float64), k.astype(np.float64)) * scale
    if causal:
        n = q.shape[2]
        s = np.where(np.tril(np.ones((n, n), bool)), s, -np.inf)
    mx = s.max(-1, keepdims=True)
    return (mx[..., 0] + np.log(np.exp(s - mx).sum(-1))).astype(F32)


# ---------------------------------------------------------------------------------------------
# Histogram — examples/09_histogram.py:17-41
# ---------------------------------------------------------------------------------------------
def histogram(x, num_bins: int, lo: float, hi: float) -> np.ndarray:
    """Counts per bin, int32.  Bin index is computed in float32, values out of range are dropped.

    Uses `np.bincount` in place of the interpreter's one-at-a-time colliding atomics
    (src/enceladus/language/ops.py:1893-1901): integer addition commutes, so the counts are the same.
    """
    inv_width = F32(num_bins / (hi - lo))  # :32 float scalar argument -> f32
    counts = np.zeros(num_bins, np.int64)
    flat = np.asarray(x).reshape(-1)
    step = 1 << 24
    for s in range(0, flat.size, step):
        xs = flat[s : s + step].astype(F32)  # :21
        t = np.floor((xs - F32(lo)) * inv_width)  # :22
        t = np.where(np.isnan(t), 0.0, t)
        bi = np.clip(t, -(2.0**31), 2.0**31 - 1).astype(np.int64)  # saturating float->int32
        bi = bi[(bi >= 0) & (bi < num_bins)]  # :23
        counts += np.bincount(bi, minlength=num_bins)
    return counts.astype(np.uint32).view(np.int32) if counts.max(initial=0) >= 2**31 else counts.astype(np.int32)


# ---------------------------------------------------------------------------------------------
# Cumulative sum — examples/10_cumsum.py:17-42, tl.cumsum src/enceladus/language/ops.py:2047-2060
# ---------------------------------------------------------------------------------------------
def cumsum_dtypes(dtype):
    """(accumulation dtype, output dtype) of `tl.cumsum` for an input dtype."""
    dtype = np.dtype(dtype)
    if dtype.kind in "iub":
        acc = np.dtype(np.int32) if dtype.itemsize < 4 and dtype.kind != "u" else dtype
        if dtype.kind == "u" and dtype.itemsize < 4:
            acc = np.dtype(np.uint32)
        if dtype.kind == "b":
            acc = np.dtype(np.int32)
        return acc, acc
    return np.dtype(F32) if dtype.itemsize < 4 or dtype.kind == "V" else dtype, dtype


def cumsum(x, reverse: bool = False) -> np.ndarray:
    """Row-wise inclusive scan of a 2-D array (or a flat scan of a 1-D one)."""
    acc, out = cumsum_dtypes(x.dtype)
    z = np.asarray(x).astype(acc)
    ax = z.ndim - 1
    if reverse:
        z = np.flip(z, ax)
    r = np.cumsum(z, axis=ax, dtype=acc)
    if reverse:
        r = np.flip(r, ax)
    return np.ascontiguousarray(r).astype(out)


def vector_add(x, y) -> np.ndarray:
    """examples/01_vector_add.py:15-22."""
    return x + y
