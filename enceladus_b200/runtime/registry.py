"""Kernel registry: kernel name + parameter list -> one typed call into the CUDA library.

The reference identifies a kernel by a specialization of its Python source
(src/enceladus/runtime/compile.py:38-47) and binds argument i to `[[buffer(i)]]`
(src/enceladus/runtime/launcher.py:457-512).  Here the kernels are the fixed set the reference ships as
examples; each adapter reads the problem out of the launch arguments the way the reference's host
wrappers pass them (softmax rows = grid[0], attention batch*heads = grid[1], ...), checks what the
launch implies (the block covers the row, the grid covers the problem) and calls the native entry
point.  An unknown kernel raises `NotImplementedError`.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

from enceladus_b200 import _native as N
from enceladus_b200.runtime import interop


@dataclass
class Split:
    """How a launch can be cut into independent pieces (rows, elements, M-blocks, (batch, head) slices).

    Used for NumPy arguments only: the launcher stages, runs and copies back one piece after the other on
    two streams (copies in and kernels on one, copies out on the other), so that the host-to-device copy
    of piece i+1 and the device-to-host copy of piece i overlap (PCIe carries both directions at once).
    Arrays that are not listed are shared by all pieces and staged once.
    """

    units: int                                   # independent units in the launch
    arrays: dict[str, int]                       # partitioned array -> elements per unit in its flat view
    grid: Callable[[int], tuple[int, int, int]]  # units in a piece -> grid of its launch
    rebind: Callable[[int], dict[str, Any]] = field(default=lambda n: {})  # units in a piece -> changed scalars
    # Pieces that are not independent but form a chain (the flat scan: every piece starts from the last value of
    # the piece before): called with the resolved arguments of a piece and of its predecessor (None for the
    # first) before the piece is launched; the pieces run in order on one stream.
    chain: Callable[[dict[str, Any], dict[str, Any] | None], None] | None = None


@dataclass
class Adapter:
    name: str
    params: tuple[str, ...]
    arrays: frozenset[str]
    outputs: frozenset[str]
    kernel_id: int
    fn: Callable[[dict[str, Any], tuple[int, int, int], int, int], None] = field(repr=False, default=None)
    # name -> number of elements the kernel writes into that output when it is laid out densely; a NumPy
    # output of exactly that size is fully overwritten, so its old contents need not be copied in
    extents: Callable[[dict[str, Any], tuple[int, int, int]], dict[str, int]] | None = field(repr=False, default=None)
    # how to cut a launch into independent pieces, or None when the kernel has no such cut
    split: Callable[[dict[str, Any], tuple[int, int, int]], Split | None] | None = field(repr=False, default=None)

    def __post_init__(self) -> None:
        self.array_list = tuple(p for p in self.params if p in self.arrays)

    def launch(self, a: dict[str, Any], grid: tuple[int, int, int], variant: int, stream: int) -> None:
        self.fn(a, grid, variant, stream)


_REGISTRY: dict[str, Adapter] = {}


def register(name: str, params: str, arrays: str, outputs: str, kernel_id: int, extents=None, split=None):
    def deco(fn):
        _REGISTRY[name] = Adapter(name, tuple(params.split()), frozenset(arrays.split()),
                                  frozenset(outputs.split()), kernel_id, fn, extents, split)
        return fn

    return deco


def lookup(name: str, params: tuple[str, ...]) -> Adapter:
    ad = _REGISTRY.get(name)
    if ad is None:
        raise NotImplementedError(
            f"kernel `{name}` has no hand-written CUDA implementation. This build runs the kernel set "
            f"{sorted(_REGISTRY)}; it has no code generator and no CPU fallback.")
    if ad.params != params:
        raise NotImplementedError(
            f"kernel `{name}` is known with parameters {ad.params}, but this definition has {params}")
    return ad


def kernels() -> list[str]:
    return sorted(_REGISTRY)


def _ptr(t: Any) -> int:
    return int(t.data_ptr())


def _code(t: Any) -> int:
    return interop.dtype_code(t)


def _same_dtype(a: dict[str, Any], *names: str) -> int:
    codes = {n: _code(a[n]) for n in names}
    if len(set(codes.values())) != 1:
        raise TypeError(f"arguments {list(names)} must share one element type, but got "
                        f"{ {n: str(interop.element_dtype(a[n])) for n in names} }")
    return next(iter(codes.values()))


def _covers(what: str, have: int, need: int) -> None:
    if have < need:
        raise NotImplementedError(
            f"{what}: the launch covers {have} but the problem needs {need}; the CUDA kernels "
            "process whole problems, so a launch must cover its arrays")


# ---- softmax_kernel(out_ptr, in_ptr, stride_in, stride_out, n_cols, BLOCK) -------------------------
@register("softmax_kernel", "out_ptr in_ptr stride_in stride_out n_cols BLOCK", "out_ptr in_ptr", "out_ptr",
          N.K_SOFTMAX,
          extents=lambda a, g: {"out_ptr": g[0] * int(a["n_cols"])} if int(a["stride_out"]) == int(a["n_cols"]) else {},
          split=lambda a, g: Split(g[0], {"in_ptr": int(a["stride_in"]), "out_ptr": int(a["stride_out"])}, lambda n: (n, 1, 1)))
def _softmax(a, grid, variant, stream):
    _covers("softmax_kernel BLOCK", int(a["BLOCK"]), int(a["n_cols"]))
    dt = _same_dtype(a, "out_ptr", "in_ptr")
    N.call("enc_softmax", _ptr(a["in_ptr"]), _ptr(a["out_ptr"]), grid[0], int(a["n_cols"]),
           int(a["stride_in"]), int(a["stride_out"]), dt, variant, stream)


# ---- layernorm_kernel(x, y, w, b, mean, rstd, stride_x, stride_y, n_cols, eps, BLOCK) --------------
@register("layernorm_kernel", "x_ptr y_ptr w_ptr b_ptr mean_ptr rstd_ptr stride_x stride_y n_cols eps BLOCK",
          "x_ptr y_ptr w_ptr b_ptr mean_ptr rstd_ptr", "y_ptr mean_ptr rstd_ptr", N.K_LAYERNORM,
          extents=lambda a, g: {"mean_ptr": g[0], "rstd_ptr": g[0], **({"y_ptr": g[0] * int(a["n_cols"])} if int(a["stride_y"]) == int(a["n_cols"]) else {})},
          split=lambda a, g: Split(g[0], {"x_ptr": int(a["stride_x"]), "y_ptr": int(a["stride_y"]), "mean_ptr": 1, "rstd_ptr": 1},
                                   lambda n: (n, 1, 1)))
def _layernorm(a, grid, variant, stream):
    dt = _same_dtype(a, "x_ptr", "y_ptr", "w_ptr", "b_ptr")
    for n in ("mean_ptr", "rstd_ptr"):
        if _code(a[n]) != N.F32:
            raise TypeError(f"argument `{n}` must be float32")
    N.call("enc_layernorm", _ptr(a["x_ptr"]), _ptr(a["y_ptr"]), _ptr(a["w_ptr"]), _ptr(a["b_ptr"]),
           _ptr(a["mean_ptr"]), _ptr(a["rstd_ptr"]), grid[0], int(a["n_cols"]), int(a["stride_x"]),
           int(a["stride_y"]), float(a["eps"]), dt, variant, stream)


# ---- rmsnorm_kernel(x, w, out, stride_x, stride_out, n_cols, eps, BLOCK) --------------------------
@register("rmsnorm_kernel", "x_ptr w_ptr out_ptr stride_x stride_out n_cols eps BLOCK", "x_ptr w_ptr out_ptr",
          "out_ptr", N.K_RMSNORM,
          extents=lambda a, g: {"out_ptr": g[0] * int(a["n_cols"])} if int(a["stride_out"]) == int(a["n_cols"]) else {},
          split=lambda a, g: Split(g[0], {"x_ptr": int(a["stride_x"]), "out_ptr": int(a["stride_out"])}, lambda n: (n, 1, 1)))
def _rmsnorm(a, grid, variant, stream):
    _covers("rmsnorm_kernel BLOCK", int(a["BLOCK"]), int(a["n_cols"]))
    dt = _same_dtype(a, "x_ptr", "w_ptr", "out_ptr")
    N.call("enc_rmsnorm", _ptr(a["x_ptr"]), _ptr(a["w_ptr"]), _ptr(a["out_ptr"]), grid[0], int(a["n_cols"]),
           int(a["stride_x"]), int(a["stride_out"]), float(a["eps"]), dt, variant, stream)


# ---- fused_gelu_kernel(x, bias, out, n, n_cols, scale, BLOCK) -------------------------------------
@register("fused_gelu_kernel", "x_ptr bias_ptr out_ptr n n_cols scale BLOCK", "x_ptr bias_ptr out_ptr", "out_ptr",
          N.K_GELU,
          extents=lambda a, g: {"out_ptr": int(a["n"])},
          # whole rows of n_cols per piece, so that the bias index (i mod n_cols) is unchanged
          split=lambda a, g: Split(int(a["n"]) // int(a["n_cols"]), {"x_ptr": int(a["n_cols"]), "out_ptr": int(a["n_cols"])},
                                   lambda n: (-(-n * int(a["n_cols"]) // int(a["BLOCK"])), 1, 1),
                                   lambda n: {"n": n * int(a["n_cols"])}) if int(a["n_cols"]) > 0 and int(a["n"]) % int(a["n_cols"]) == 0 else None)
def _fused_gelu(a, grid, variant, stream):
    n = int(a["n"])
    _covers("fused_gelu_kernel grid*BLOCK", grid[0] * int(a["BLOCK"]), n)
    dt = _same_dtype(a, "x_ptr", "bias_ptr", "out_ptr")
    N.call("enc_gelu", _ptr(a["x_ptr"]), _ptr(a["bias_ptr"]), _ptr(a["out_ptr"]), n, int(a["n_cols"]),
           float(a["scale"]), 1, 0, dt, variant, stream)


# ---- tanh_gelu_kernel(x, out, n, BLOCK): the tanh form of benchmark config 2 ----------------------
@register("tanh_gelu_kernel", "x_ptr out_ptr n BLOCK", "x_ptr out_ptr", "out_ptr", N.K_GELU,
          extents=lambda a, g: {"out_ptr": int(a["n"])},
          split=lambda a, g: Split(int(a["n"]), {"x_ptr": 1, "out_ptr": 1}, lambda n: (-(-n // int(a["BLOCK"])), 1, 1),
                                   lambda n: {"n": n}))
def _tanh_gelu(a, grid, variant, stream):
    n = int(a["n"])
    _covers("tanh_gelu_kernel grid*BLOCK", grid[0] * int(a["BLOCK"]), n)
    dt = _same_dtype(a, "x_ptr", "out_ptr")
    N.call("enc_gelu", _ptr(a["x_ptr"]), None, _ptr(a["out_ptr"]), n, 0, 1.0, 0, 1, dt, variant, stream)


# ---- add_kernel(x, y, out, n, BLOCK) -------------------------------------------------------------
@register("add_kernel", "x_ptr y_ptr out_ptr n BLOCK", "x_ptr y_ptr out_ptr", "out_ptr", N.K_ADD,
          extents=lambda a, g: {"out_ptr": int(a["n"])},
          split=lambda a, g: Split(int(a["n"]), {"x_ptr": 1, "y_ptr": 1, "out_ptr": 1}, lambda n: (-(-n // int(a["BLOCK"])), 1, 1),
                                   lambda n: {"n": n}))
def _add(a, grid, variant, stream):
    n = int(a["n"])
    _covers("add_kernel grid*BLOCK", grid[0] * int(a["BLOCK"]), n)
    dt = _same_dtype(a, "x_ptr", "y_ptr", "out_ptr")
    N.call("enc_add", _ptr(a["x_ptr"]), _ptr(a["y_ptr"]), _ptr(a["out_ptr"]), n, dt, variant, stream)


# ---- histogram_kernel(x, hist, n, lo, inv_width, NUM_BINS, BLOCK) ---------------------------------
@register("histogram_kernel", "x_ptr hist_ptr n lo inv_width NUM_BINS BLOCK", "x_ptr hist_ptr", "hist_ptr",
          N.K_HISTOGRAM)
def _histogram(a, grid, variant, stream):
    n = int(a["n"])
    _covers("histogram_kernel grid*BLOCK", grid[0] * int(a["BLOCK"]), n)
    if _code(a["hist_ptr"]) != N.I32:
        raise TypeError("argument `hist_ptr` must be int32")
    N.call("enc_histogram", _ptr(a["x_ptr"]), _ptr(a["hist_ptr"]), n, float(a["lo"]), float(a["inv_width"]),
           int(a["NUM_BINS"]), _code(a["x_ptr"]), variant, stream)


# ---- cumsum_kernel(out, in, n_rows, n_cols, stride_in, stride_out, REVERSE, BLOCK_M, BLOCK_N) -----
def _cumsum_split(a, g):
    """The flat forward scan cut along the row: a piece is seeded with the last output of the piece before it
    (the accumulator itself for int32 and float32 outputs, the types the kernel takes a seed for; float16 /
    bfloat16 outputs are rounded, so those stay in one piece, and so do the other integer widths).  Integer
    results are the one-piece results bit for bit; float32 results differ from
    them in the order of the additions, as the one-piece scan's own tile order does from a sequential sum."""
    if int(a["n_rows"]) != 1 or bool(a["REVERSE"]):
        return None
    if _code(a["in_ptr"]) not in (N.I32, N.F32) or _code(a["out_ptr"]) != _code(a["in_ptr"]):
        return None

    def chain(piece, before):
        piece["_seed"] = None if before is None else before["out_ptr"][-1:]

    return Split(int(a["n_cols"]), {"in_ptr": 1, "out_ptr": 1}, lambda n: (1, 1, 1),
                 lambda n: {"n_cols": int(n), "stride_in": int(n), "stride_out": int(n), "BLOCK_N": 1 << max(0, (int(n) - 1).bit_length())},
                 chain)


@register("cumsum_kernel", "out_ptr in_ptr n_rows n_cols stride_in stride_out REVERSE BLOCK_M BLOCK_N",
          "out_ptr in_ptr", "out_ptr", N.K_CUMSUM,
          extents=lambda a, g: {"out_ptr": int(a["n_rows"]) * int(a["n_cols"])} if int(a["stride_out"]) == int(a["n_cols"]) or int(a["n_rows"]) == 1 else {},
          split=_cumsum_split)
def _cumsum(a, grid, variant, stream):
    rows, cols = int(a["n_rows"]), int(a["n_cols"])
    _covers("cumsum_kernel BLOCK_N", int(a["BLOCK_N"]), cols)
    _covers("cumsum_kernel grid*BLOCK_M", grid[0] * int(a["BLOCK_M"]), rows)
    dt = _code(a["in_ptr"])
    want = N.load().enc_cumsum_out_dtype(dt)
    if want < 0:
        raise TypeError(f"cumsum doesn't support element type {interop.element_dtype(a['in_ptr'])}")
    if _code(a["out_ptr"]) != want:
        raise TypeError(f"cumsum of {interop.element_dtype(a['in_ptr'])} writes "
                        f"{'int32' if want == N.I32 else interop.element_dtype(a['in_ptr'])}, but `out_ptr` is "
                        f"{interop.element_dtype(a['out_ptr'])}")
    seed = a.get("_seed")  # set by the chained staging of a long NumPy row only
    N.call("enc_cumsum", _ptr(a["in_ptr"]), _ptr(a["out_ptr"]), rows, cols, int(a["stride_in"]),
           int(a["stride_out"]), int(bool(a["REVERSE"])), dt, None if seed is None else _ptr(seed), variant, stream)


# ---- matmul kernels -------------------------------------------------------------------------------
def _matmul_split(a, g):
    """Pieces of whole rows of A and C; B (and the bias) are shared."""
    return Split(int(a["M"]), {"a_ptr": int(a["stride_am"]), "c_ptr": int(a["stride_cm"])},
                 lambda n: (g[0], -(-n // int(a["BM"])), 1), lambda n: {"M": n})


def _matmul_common(a, grid, variant, stream, bias, epilogue):
    m, n, k = int(a["M"]), int(a["N"]), int(a["K"])
    _covers("matmul grid[0]*BN", grid[0] * int(a["BN"]), n)
    _covers("matmul grid[1]*BM", grid[1] * int(a["BM"]), m)
    names = ("a_ptr", "b_ptr", "c_ptr") + (("bias_ptr",) if bias else ())
    dt = _same_dtype(a, *names)
    N.call("enc_matmul", _ptr(a["a_ptr"]), _ptr(a["b_ptr"]), _ptr(a["bias_ptr"]) if bias else None,
           _ptr(a["c_ptr"]), m, n, k, int(a["stride_am"]), int(a["stride_bk"]), int(a["stride_cm"]), epilogue,
           dt, variant, stream)


@register("matmul_bias_gelu_kernel", "a_ptr b_ptr bias_ptr c_ptr M N K stride_am stride_bk stride_cm BM BN BK",
          "a_ptr b_ptr bias_ptr c_ptr", "c_ptr", N.K_MATMUL,
          extents=lambda a, g: {"c_ptr": int(a["M"]) * int(a["N"])} if int(a["stride_cm"]) == int(a["N"]) else {},
          split=_matmul_split)
def _matmul_bias_gelu(a, grid, variant, stream):
    _matmul_common(a, grid, variant, stream, bias=True, epilogue=1)


@register("matmul_desc_kernel", "a_ptr b_ptr c_ptr M N K stride_am stride_bk stride_cm BM BN BK",
          "a_ptr b_ptr c_ptr", "c_ptr", N.K_MATMUL,
          extents=lambda a, g: {"c_ptr": int(a["M"]) * int(a["N"])} if int(a["stride_cm"]) == int(a["N"]) else {},
          split=_matmul_split)
def _matmul_desc(a, grid, variant, stream):
    _matmul_common(a, grid, variant, stream, bias=False, epilogue=0)


@register("matmul_kernel",
          "a_ptr b_ptr c_ptr M N K stride_am stride_ak stride_bk stride_bn stride_cm stride_cn BM BN BK",
          "a_ptr b_ptr c_ptr", "c_ptr", N.K_MATMUL,
          extents=lambda a, g: {"c_ptr": int(a["M"]) * int(a["N"])} if int(a["stride_cm"]) == int(a["N"]) else {},
          split=_matmul_split)
def _matmul_ptr(a, grid, variant, stream):
    for s in ("stride_ak", "stride_bn", "stride_cn"):
        if int(a[s]) != 1:
            raise NotImplementedError(f"matmul_kernel: {s} = {a[s]}; the CUDA matmul needs unit inner strides")
    _matmul_common(a, grid, variant, stream, bias=False, epilogue=0)


# ---- int8_matmul_kernel(a, b, c, M, N, K, BM, BN, BK): dense row-major integer operands, int32 result -------
@register("int8_matmul_kernel", "a_ptr b_ptr c_ptr M N K BM BN BK", "a_ptr b_ptr c_ptr", "c_ptr", N.K_MATMUL_INT,
          extents=lambda a, g: {"c_ptr": int(a["M"]) * int(a["N"])},
          split=lambda a, g: Split(int(a["M"]), {"a_ptr": int(a["K"]), "c_ptr": int(a["N"])},
                                   lambda n: (g[0], -(-n // int(a["BM"])), 1), lambda n: {"M": n}))
def _int_matmul(a, grid, variant, stream):
    m, n, k = int(a["M"]), int(a["N"]), int(a["K"])
    _covers("int8_matmul_kernel grid[0]*BN", grid[0] * int(a["BN"]), n)
    _covers("int8_matmul_kernel grid[1]*BM", grid[1] * int(a["BM"]), m)
    dt = _same_dtype(a, "a_ptr", "b_ptr")
    if dt not in (N.I8, N.U8, N.I16, N.I32):
        raise TypeError(f"int8_matmul_kernel takes int8, uint8, int16 or int32 operands, not {interop.element_dtype(a['a_ptr'])}")
    if _code(a["c_ptr"]) != N.I32:
        raise TypeError("argument `c_ptr` must be int32")
    N.call("enc_matmul_int", _ptr(a["a_ptr"]), _ptr(a["b_ptr"]), _ptr(a["c_ptr"]), m, n, k, k, n, n, dt, variant, stream)


# ---- attention_kernel(q, k, v, o, sm_scale, N_CTX, stride_h, stride_m, HEAD_DIM, BLOCK_M, BLOCK_N, CAUSAL)
@register("attention_kernel",
          "q_ptr k_ptr v_ptr o_ptr sm_scale N_CTX stride_h stride_m HEAD_DIM BLOCK_M BLOCK_N CAUSAL",
          "q_ptr k_ptr v_ptr o_ptr", "o_ptr", N.K_ATTENTION,
          extents=lambda a, g: {"o_ptr": g[1] * int(a["N_CTX"]) * int(a["HEAD_DIM"]), "lse_ptr": g[1] * int(a["N_CTX"])} if int(a["stride_m"]) == int(a["HEAD_DIM"]) and int(a["stride_h"]) == int(a["N_CTX"]) * int(a["HEAD_DIM"]) else {},
          split=lambda a, g: Split(g[1], {n: int(a["stride_h"]) for n in ("q_ptr", "k_ptr", "v_ptr", "o_ptr")}, lambda n: (g[0], n, 1)))
def _attention(a, grid, variant, stream):
    s = int(a["N_CTX"])
    _covers("attention_kernel grid[0]*BLOCK_M", grid[0] * int(a["BLOCK_M"]), s)
    dt = _same_dtype(a, "q_ptr", "k_ptr", "v_ptr", "o_ptr")
    N.call("enc_attention_fwd", _ptr(a["q_ptr"]), _ptr(a["k_ptr"]), _ptr(a["v_ptr"]), _ptr(a["o_ptr"]), None,
           grid[1], s, int(a["HEAD_DIM"]), int(a["stride_h"]), int(a["stride_m"]), float(a["sm_scale"]),
           int(bool(a["CAUSAL"])), dt, variant, stream)


# The same kernel with one more output: float32 logsumexp [batch*heads, seq] of the running statistics.
@register("attention_lse_kernel",
          "q_ptr k_ptr v_ptr o_ptr lse_ptr sm_scale N_CTX stride_h stride_m HEAD_DIM BLOCK_M BLOCK_N CAUSAL",
          "q_ptr k_ptr v_ptr o_ptr lse_ptr", "o_ptr lse_ptr", N.K_ATTENTION,
          extents=lambda a, g: {"o_ptr": g[1] * int(a["N_CTX"]) * int(a["HEAD_DIM"]), "lse_ptr": g[1] * int(a["N_CTX"])} if int(a["stride_m"]) == int(a["HEAD_DIM"]) and int(a["stride_h"]) == int(a["N_CTX"]) * int(a["HEAD_DIM"]) else {},
          split=lambda a, g: Split(g[1], {**{n: int(a["stride_h"]) for n in ("q_ptr", "k_ptr", "v_ptr", "o_ptr")}, "lse_ptr": int(a["N_CTX"])},
                                   lambda n: (g[0], n, 1)))
def _attention_lse(a, grid, variant, stream):
    s = int(a["N_CTX"])
    _covers("attention_lse_kernel grid[0]*BLOCK_M", grid[0] * int(a["BLOCK_M"]), s)
    dt = _same_dtype(a, "q_ptr", "k_ptr", "v_ptr", "o_ptr")
    if _code(a["lse_ptr"]) != N.F32:
        raise TypeError("argument `lse_ptr` must be float32")
    N.call("enc_attention_fwd", _ptr(a["q_ptr"]), _ptr(a["k_ptr"]), _ptr(a["v_ptr"]), _ptr(a["o_ptr"]),
           _ptr(a["lse_ptr"]), grid[1], s, int(a["HEAD_DIM"]), int(a["stride_h"]), int(a["stride_m"]),
           float(a["sm_scale"]), int(bool(a["CAUSAL"])), dt, variant, stream)


