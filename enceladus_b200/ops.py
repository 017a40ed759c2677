"""The kernel set: `@jit` kernel definitions and their host wrappers.

Each wrapper has the signature and behaviour of the reference example of the same name
(examples/01_vector_add.py ... examples/10_cumsum.py): it accepts NumPy arrays or torch CUDA tensors,
allocates its outputs with `new_empty`/`new_zeros` and launches `kernel[grid](...)` with the same
arguments.  The kernel bodies are not executed — each launch is served by the hand-written CUDA kernel
registered under the kernel's name — so a body here is only a statement of what that kernel computes.
A user's own copy of a reference example works the same way after `import enceladus_b200 as enceladus`.
"""

from __future__ import annotations

import math

import numpy as np

import enceladus_b200 as enceladus
import enceladus_b200.language as tl
from enceladus_b200.configs import attention_configs, matmul_configs


# ---- 01 vector add -----------------------------------------------------------------------------
@enceladus.jit
def add_kernel(x_ptr, y_ptr, out_ptr, n, BLOCK: tl.constexpr):
    """out[i] = x[i] + y[i] for i < n."""


def add(x, y, block: int = 1024):
    """Returns `x + y` for two contiguous arrays of the same shape and dtype."""
    out = enceladus.new_empty(x)
    n = int(np.prod(x.shape))
    add_kernel[(enceladus.cdiv(n, block),)](x, y, out, n, BLOCK=block)
    return out


# ---- 02 softmax --------------------------------------------------------------------------------
@enceladus.jit
def softmax_kernel(out_ptr, in_ptr, stride_in, stride_out, n_cols, BLOCK: tl.constexpr):
    """One row per program: exp(x - max(x)) / sum(exp(x - max(x))) in float32, stored in the input dtype."""


def softmax(x):
    """Returns the softmax of each row of a 2D array, in the input dtype.

    The rows can be strided, but the elements within a row must be contiguous.
    """
    m, n = x.shape
    out = enceladus.new_empty(x)
    softmax_kernel[(m,)](out, x, enceladus.element_strides(x)[0], enceladus.element_strides(out)[0], n,
                         BLOCK=enceladus.next_power_of_2(n))
    return out


# ---- 03 layernorm ------------------------------------------------------------------------------
@enceladus.jit
def layernorm_kernel(x_ptr, y_ptr, w_ptr, b_ptr, mean_ptr, rstd_ptr, stride_x, stride_y, n_cols, eps,
                     BLOCK: tl.constexpr):
    """One row per program: mean, centred variance, rstd = 1/sqrt(var+eps); y = (x-mean)*rstd*w + b."""


def layernorm(x, w, b, eps: float = 1e-5, block: int | None = None):
    """Returns `(y, mean, rstd)` for a 2D input normalized over its last dimension."""
    m, n = x.shape
    y = enceladus.new_empty(x)
    mean = enceladus.new_empty(x, (m,), np.float32)
    rstd = enceladus.new_empty(x, (m,), np.float32)
    block = block or min(1024, enceladus.next_power_of_2(n))
    stride_x, stride_y = enceladus.element_strides(x)[0], enceladus.element_strides(y)[0]
    layernorm_kernel[(m,)](x, y, w, b, mean, rstd, stride_x, stride_y, n, eps, BLOCK=block)
    return y, mean, rstd


# ---- 05 fused GELU -----------------------------------------------------------------------------
@enceladus.jit
def fused_gelu_kernel(x_ptr, bias_ptr, out_ptr, n, n_cols, scale, BLOCK: tl.constexpr):
    """t = x*scale + bias[i % n_cols]; out = 0.5*t*(1 + erf(t/sqrt(2)))."""


def fused_gelu(x, bias, scale: float, block: int = 1024):
    """Returns `gelu(x * scale + bias)` for a contiguous 2D `x` and a bias per column."""
    out = enceladus.new_empty(x)
    n = int(np.prod(x.shape))
    fused_gelu_kernel[(enceladus.cdiv(n, block),)](x, bias, out, n, x.shape[-1], scale, BLOCK=block)
    return out


@enceladus.jit
def tanh_gelu_kernel(x_ptr, out_ptr, n, BLOCK: tl.constexpr):
    """out = 0.5*x*(1 + tanh(0.7978845608*(x + 0.044715*x^3))), elementwise."""


def tanh_gelu(x, block: int = 1024):
    """Returns the tanh-form GELU of a contiguous array of any shape."""
    out = enceladus.new_empty(x)
    n = int(np.prod(x.shape))
    tanh_gelu_kernel[(enceladus.cdiv(n, block),)](x, out, n, BLOCK=block)
    return out


# ---- 06 rmsnorm --------------------------------------------------------------------------------
@enceladus.jit
def rmsnorm_kernel(x_ptr, w_ptr, out_ptr, stride_x, stride_out, n_cols, eps, BLOCK: tl.constexpr):
    """One row per program: x * (1/sqrt(mean(x^2) + eps)) * w."""


def rmsnorm(x, w, eps: float = 1e-6):
    """Returns RMSNorm of each row of a 2D array, in the input dtype."""
    m, n = x.shape
    out = enceladus.new_empty(x)
    rmsnorm_kernel[(m,)](x, w, out, enceladus.element_strides(x)[0], enceladus.element_strides(out)[0], n, eps,
                         BLOCK=enceladus.next_power_of_2(n))
    return out


# ---- 04 / 07 matmul ----------------------------------------------------------------------------
@enceladus.jit
def matmul_desc_kernel(a_ptr, b_ptr, c_ptr, M, N, K, stride_am, stride_bk, stride_cm, BM: tl.constexpr,
                       BN: tl.constexpr, BK: tl.constexpr):
    """C = A @ B with float32 accumulation; out-of-range tile elements read as zero, are not stored."""


@enceladus.jit
def matmul_bias_gelu_kernel(a_ptr, b_ptr, bias_ptr, c_ptr, M, N, K, stride_am, stride_bk, stride_cm,
                            BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
    """C = gelu_erf(A @ B + bias[None, :]) with the epilogue applied to the float32 accumulator."""


def matmul_desc(a, b, c=None, bm: int = 128, bn: int = 256, bk: int = 64, num_warps: int = 4,
                dot_backend: str = "auto"):
    """Returns `a @ b` in the input dtype. `a`, `b`, and `c` must be row-major."""
    (m, k), (_, n) = a.shape, b.shape
    if c is None:
        c = enceladus.new_empty(a, (m, n))
    grid = (enceladus.cdiv(n, bn), enceladus.cdiv(m, bm))
    sa, sb, sc = (enceladus.element_strides(t)[0] for t in (a, b, c))
    matmul_desc_kernel[grid](a, b, c, m, n, k, sa, sb, sc, BM=bm, BN=bn, BK=bk, num_warps=num_warps,
                             dot_backend=dot_backend)
    return c


matmul = matmul_desc


def matmul_bias_gelu(a, b, bias, c=None, bm: int = 128, bn: int = 256, bk: int = 64, dot_backend: str = "auto"):
    """Returns `gelu(a @ b + bias)` in the input dtype."""
    (m, k), (_, n) = a.shape, b.shape
    if c is None:
        c = enceladus.new_empty(a, (m, n))
    grid = (enceladus.cdiv(n, bn), enceladus.cdiv(m, bm))
    sa, sb, sc = (enceladus.element_strides(t)[0] for t in (a, b, c))
    matmul_bias_gelu_kernel[grid](a, b, bias, c, m, n, k, sa, sb, sc, BM=bm, BN=bn, BK=bk, dot_backend=dot_backend)
    return c


matmul_desc_tuned = enceladus.autotune(configs=matmul_configs("float16"), key=["M", "N", "K"])(matmul_desc_kernel)


def matmul_tuned(a, b, c=None):
    """Returns `a @ b` using the fastest tile variant for this shape and dtype."""
    (m, k), (_, n) = a.shape, b.shape
    if c is None:
        c = enceladus.new_empty(a, (m, n))
    grid = lambda meta: (enceladus.cdiv(n, meta["BN"]), enceladus.cdiv(m, meta["BM"]))  # noqa: E731
    sa, sb, sc = (enceladus.element_strides(t)[0] for t in (a, b, c))
    matmul_desc_tuned[grid](a, b, c, m, n, k, sa, sb, sc)
    return c


# ---- integer matmul (benchmarks/bench_matmul.py:100-131) ------------------------------------------
@enceladus.jit
def int8_matmul_kernel(a_ptr, b_ptr, c_ptr, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
    """C[int32] = A @ B for dense row-major integer A [M, K] and B [K, N]: int32 accumulation, exact, products
    and sums wrap modulo 2^32 (an integer `tl.dot` per K block)."""


def int_matmul(a, b, c=None, bm: int = 128, bn: int = 256, bk: int = 128):
    """Returns the exact int32 product of two contiguous integer matrices (int8, uint8, int16 or int32)."""
    (m, k), (_, n) = a.shape, b.shape
    if c is None:
        c = enceladus.new_empty(a, (m, n), np.int32)
    int8_matmul_kernel[(enceladus.cdiv(n, bn), enceladus.cdiv(m, bm))](a, b, c, m, n, k, BM=bm, BN=bn, BK=bk)
    return c


# ---- 08 flash attention ------------------------------------------------------------------------
@enceladus.jit
def attention_kernel(q_ptr, k_ptr, v_ptr, o_ptr, sm_scale, N_CTX, stride_h, stride_m, HEAD_DIM: tl.constexpr,
                     BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, CAUSAL: tl.constexpr):
    """softmax(q k^T * sm_scale [causal]) v per (batch, head): base-2 online softmax in float32, the
    probabilities rounded to the input dtype before the second product."""


@enceladus.jit
def attention_lse_kernel(q_ptr, k_ptr, v_ptr, o_ptr, lse_ptr, sm_scale, N_CTX, stride_h, stride_m,
                         HEAD_DIM: tl.constexpr, BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr,
                         CAUSAL: tl.constexpr):
    """attention_kernel plus lse[b*h, i] = ln2 * (m_i + log2 l_i) of the running statistics, float32."""


def _check_qkv(q, k, v):
    if not (tuple(q.shape) == tuple(k.shape) == tuple(v.shape)) or len(q.shape) != 4:
        raise ValueError("q, k, and v must all have shape (batch, heads, seq_len, head_dim)")
    if q.shape[-1] not in (16, 32, 64, 128):
        raise ValueError(f"head_dim must be 16, 32, 64, or 128, not {q.shape[-1]}")


def attention(q, k, v, causal: bool = False, sm_scale: float | None = None, o=None, block_m: int = 128,
              block_n: int = 128, num_warps: int = 4, return_lse: bool = False):
    """Returns `softmax(q @ k^T * sm_scale) @ v` for contiguous (batch, heads, seq, dim) inputs.

    With `return_lse=True`, also returns the float32 log-sum-exp of the scaled scores, shape
    (batch, heads, seq).
    """
    _check_qkv(q, k, v)
    z, h, n, d = q.shape
    o = enceladus.new_empty(q) if o is None else o
    scale = 1.0 / math.sqrt(d) if sm_scale is None else sm_scale
    grid = (enceladus.cdiv(n, block_m), z * h)
    if return_lse:
        lse = enceladus.new_empty(q, (z, h, n), np.float32)
        attention_lse_kernel[grid](q, k, v, o, lse, scale, n, n * d, d, HEAD_DIM=d, BLOCK_M=block_m,
                                   BLOCK_N=block_n, CAUSAL=causal, num_warps=num_warps, dot_warps=(num_warps, 1))
        return o, lse
    attention_kernel[grid](q, k, v, o, scale, n, n * d, d, HEAD_DIM=d, BLOCK_M=block_m, BLOCK_N=block_n,
                           CAUSAL=causal, num_warps=num_warps, dot_warps=(num_warps, 1))
    return o


attention_tuned_kernel = enceladus.autotune(configs=attention_configs("float16", 128),
                                            key=["N_CTX", "HEAD_DIM", "CAUSAL"])(attention_kernel)


def attention_tuned(q, k, v, causal: bool = False, sm_scale: float | None = None, o=None):
    """Returns the same result as `attention`, using the fastest tile variant for the shape."""
    _check_qkv(q, k, v)
    z, h, n, d = q.shape
    o = enceladus.new_empty(q) if o is None else o
    scale = 1.0 / math.sqrt(d) if sm_scale is None else sm_scale
    grid = lambda meta: (enceladus.cdiv(n, meta["BLOCK_M"]), z * h)  # noqa: E731
    attention_tuned_kernel[grid](q, k, v, o, scale, n, n * d, d, HEAD_DIM=d, CAUSAL=causal)
    return o


# ---- 09 histogram ------------------------------------------------------------------------------
@enceladus.jit
def histogram_kernel(x_ptr, hist_ptr, n, lo, inv_width, NUM_BINS: tl.constexpr, BLOCK: tl.constexpr):
    """hist[floor((float(x) - lo) * inv_width)] += 1 for every in-range element."""


def histogram(x, num_bins: int, lo: float, hi: float, block: int = 1024):
    """Returns the `int32` counts of `x` in `num_bins` equal bins over `[lo, hi)`."""
    hist = enceladus.new_zeros(x, (num_bins,), np.int32)
    n = int(np.prod(x.shape))
    histogram_kernel[(enceladus.cdiv(n, block),)](x, hist, n, float(lo), num_bins / (hi - lo),
                                                  NUM_BINS=num_bins, BLOCK=block)
    return hist


# ---- 10 cumsum ---------------------------------------------------------------------------------
@enceladus.jit
def cumsum_kernel(out_ptr, in_ptr, n_rows, n_cols, stride_in, stride_out, REVERSE: tl.constexpr,
                  BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr):
    """Inclusive scan of each row (suffix sums when REVERSE); narrow integers sum in int32."""


def cumsum(x, reverse: bool = False):
    """Returns the cumulative sum of each row of a 2D array, or of a 1D array of any length.

    Integers narrower than 32 bits sum in `int32`; int32 sums wrap modulo 2**32.
    """
    flat = len(x.shape) == 1
    m, n = (1, x.shape[0]) if flat else x.shape
    dt = enceladus.element_dtype(x)
    out = enceladus.new_empty(x, dtype=np.int32 if dt.kind in "iub" and dt.itemsize < 4 else dt)
    block_n = enceladus.next_power_of_2(n)
    block_m = max(1, min(16, 4096 // block_n))
    si = n if flat else enceladus.element_strides(x)[0]
    so = n if flat else enceladus.element_strides(out)[0]
    cumsum_kernel[(enceladus.cdiv(m, block_m),)](out, x, m, n, si, so, REVERSE=reverse, BLOCK_M=block_m,
                                                 BLOCK_N=block_n)
    return out
