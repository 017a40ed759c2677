"""`@jit` kernels and the `kernel[grid](...)` launch path.

Keeps the launch contract of the reference's `JITFunction` (src/enceladus/runtime/jit.py:214-418):
the signature splits into runtime and `tl.constexpr` parameters, `kernel[grid](*args, **meta)` binds
them, `grid` is a tuple of 1 to 3 ints or a callable of the argument dict, the launch options
`num_warps / num_stages / dot_warps / dot_backend` are accepted, a zero in the grid is a silent no-op.

What changes is what a launch does.  The reference compiles the Python body to Metal; here the body is
never run.  The kernel's name and parameter list select an adapter in `registry.py`, which recovers the
problem from the launch arguments exactly as the reference's host wrappers pass them and makes one call
into the CUDA library.  A kernel that is not in the registry raises: there is no code generator, no
interpreter and no CPU fallback in this build.
"""

from __future__ import annotations

import ast
import functools
import hashlib
import inspect
import os
import textwrap
import warnings
from collections.abc import Callable, Iterable, Mapping
from dataclasses import dataclass
from typing import Any

import numpy as np

from enceladus_b200 import language as tl
from enceladus_b200 import _native as N
from enceladus_b200.runtime import interop

MAX_GRID = (2**31 - 1, 65535, 65535)
_LAUNCH_OPTIONS = ("num_warps", "num_stages", "dot_warps", "dot_backend")


def cdiv(x: int, div: int) -> int:
    """Returns `ceil(x / div)` for positive integers: the number of blocks that cover `x`."""
    return -(-x // div)


def next_power_of_2(n: int) -> int:
    """Returns the smallest power of two that's greater than or equal to `n`."""
    return 1 if n <= 1 else 1 << (int(n) - 1).bit_length()


_GRID_RANK_MSG = "the grid needs 1 to 3 dimensions, but got {}. Pass a tuple such as `(n,)` or `(m, n)`."


def resolve_grid(grid: Any, bound: Mapping[str, Any]) -> tuple[int, int, int]:
    """Grid tuple from a tuple/int or a callable of the argument dict (jit.py:669-678)."""
    g = grid(dict(bound)) if callable(grid) else grid
    if isinstance(g, (int, np.integer)):
        g = (g,)
    g = tuple(int(x) for x in g)
    if not 1 <= len(g) <= 3:
        raise ValueError(_GRID_RANK_MSG.format(g))
    if any(x < 0 for x in g):
        raise ValueError(f"grid dimensions can't be negative, but got {g}")
    g = (*g, *(1,) * (3 - len(g)))
    for i, (x, lim) in enumerate(zip(g, MAX_GRID)):
        if x > lim:
            raise ValueError(f"grid dimension {i} is {x}, but the limit is {lim}")
    return g  # type: ignore[return-value]


def fingerprint_of_def(node: ast.FunctionDef) -> str | None:
    """SHA-256 of a function's normalised body, or None when the body only documents the kernel (a docstring,
    `pass`, `...`).  Normalised = the AST of the statements without the docstring and without positions, so
    comments, blank lines and line breaks do not change it; names and constants do."""
    body = list(node.body)
    if body and isinstance(body[0], ast.Expr) and isinstance(getattr(body[0], "value", None), ast.Constant) \
            and isinstance(body[0].value.value, str):
        body = body[1:]
    body = [b for b in body if not isinstance(b, ast.Pass)
            and not (isinstance(b, ast.Expr) and isinstance(b.value, ast.Constant) and b.value.value is Ellipsis)]
    if not body:
        return None
    text = "\n".join(ast.dump(b, annotate_fields=True, include_attributes=False) for b in body)
    return hashlib.sha256(text.encode()).hexdigest()


def body_fingerprint(fn: Callable[..., Any]) -> str | None:
    """`fingerprint_of_def` of a live function; raises OSError when its source cannot be read."""
    tree = ast.parse(textwrap.dedent(inspect.getsource(fn)))
    node = next(n for n in ast.walk(tree) if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef)))
    return fingerprint_of_def(node)


def check_body(fn: Callable[..., Any], name: str) -> None:
    """A `@jit` definition is served by the hand-written kernel registered under its name.  That is only right
    if the body says the same thing: either nothing (docstring / `pass`) or exactly one of the reference's own
    kernels of that name.  Anything else is refused: the reference would have compiled what the user wrote."""
    try:
        fp = body_fingerprint(fn)
    except (OSError, TypeError, SyntaxError, StopIteration):
        warnings.warn(f"kernel `{name}`: the source of this definition cannot be read, so its body cannot be "
                      "compared with the built-in CUDA kernel that will run in its place", RuntimeWarning, stacklevel=4)
        return
    if fp is None:
        return
    from enceladus_b200.runtime.kernel_bodies import KNOWN_BODIES

    if fp not in KNOWN_BODIES.get(name, ()):
        raise NotImplementedError(
            f"kernel `{name}` has a body that is not the reference's kernel of that name. This build does not "
            "compile kernel bodies: a launch of this name runs the hand-written CUDA kernel, which would ignore "
            "what the body says. Rename the kernel if it computes something else, or leave the body empty "
            "(a docstring or `pass`) to use the built-in kernel.")


@dataclass
class KernelParam:
    name: str
    index: int
    is_constexpr: bool
    default: Any
    do_not_specialize: bool


class JITFunction:
    """A kernel created by `@enceladus_b200.jit`.

    Launch it with `kernel[grid](*args, **constexprs, num_warps=4)`.
    """

    _is_enceladus_jit = True

    def __init__(self, fn: Callable[..., Any], *, interpret: bool | None = None,
                 do_not_specialize: Iterable[str | int] = (), math_mode: str = "relaxed") -> None:
        if not inspect.isfunction(fn):
            raise TypeError(f"@enceladus.jit needs a function, but got {type(fn).__name__}")
        if math_mode not in ("relaxed", "fast"):
            raise ValueError(f"math_mode must be one of ('relaxed', 'fast'), but got {math_mode!r}")
        self.fn = fn
        functools.update_wrapper(self, fn)
        self.interpret = interpret
        self.math_mode = math_mode
        self.signature = inspect.signature(fn)
        names = list(self.signature.parameters)
        dns: set[str] = set()
        for d in do_not_specialize:
            if isinstance(d, int):
                if not 0 <= d < len(names):
                    raise ValueError(f"do_not_specialize index {d} is out of range")
                d = names[d]
            if d not in names:
                raise ValueError(f"do_not_specialize names unknown parameter {d!r}")
            dns.add(d)
        params = []
        for i, (n, p) in enumerate(self.signature.parameters.items()):
            if p.kind in (p.VAR_POSITIONAL, p.VAR_KEYWORD):
                raise TypeError(f"kernel `{fn.__name__}` can't take *args or **kwargs. List every "
                                "parameter by name.")
            params.append(KernelParam(n, i, tl.is_constexpr_annotation(p.annotation), p.default, n in dns))
        self.params: list[KernelParam] = params
        self.arg_names = names
        self._constexpr_names = [p.name for p in params if p.is_constexpr]
        self._adapter = None
        self.variant: int | None = None  # forced tile variant (None = the library's choice)
        self.last_launch: dict[str, Any] = {}

    def __repr__(self) -> str:
        return f"JITFunction({self.__module__}:{self.__qualname__})"

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        raise RuntimeError(f"`{self.__name__}` is a @enceladus.jit function. Launch it with "
                           f"`{self.__name__}[grid](...)`.")

    def __getitem__(self, grid: Any) -> Callable[..., None]:
        return lambda *args, **kwargs: self.run(*args, grid=grid, **kwargs)

    def bind(self, args: tuple[Any, ...], kwargs: Mapping[str, Any]) -> dict[str, Any]:
        """Binds launch arguments to parameter names, applying defaults."""
        try:
            ba = self.signature.bind(*args, **kwargs)
        except TypeError as e:
            raise TypeError(f"{self.__name__}: {e}") from None
        ba.apply_defaults()
        return dict(ba.arguments)

    def adapter(self):
        """The registry entry that implements this kernel; raises if there is none, or if this definition's
        body is code that is not the reference's kernel of that name (the body is never executed, so serving
        it with the built-in kernel would silently compute something else)."""
        if self._adapter is None:
            from enceladus_b200.runtime import registry

            ad = registry.lookup(self.__name__, tuple(self.arg_names))
            check_body(self.fn, ad.name)
            self._adapter = ad
        return self._adapter

    def run(self, *args: Any, grid: Any, num_warps: int = 4, num_stages: int | None = None,
            dot_warps: tuple[int, int] | None = None, dot_backend: str = "auto",
            variant: int | None = None, **kwargs: Any) -> None:
        """Launches the kernel.

        `num_warps`, `num_stages`, `dot_warps` and `dot_backend` are accepted because the reference's
        host wrappers pass them (examples/07_matmul_fused.py:46-47, examples/08_flash_attention.py:101-103);
        they describe Apple SIMD-group layouts and do not affect the CUDA kernels.  `variant` picks one
        of the hand-written tile variants of the kernel (the autotuner uses it).
        """
        interpret = self.interpret
        if interpret is None:
            interpret = os.environ.get("ENCELADUS_INTERPRET", "0") not in ("", "0")
        if interpret:
            raise RuntimeError(
                "ENCELADUS_INTERPRET / interpret=True asks for the reference's CPU interpreter, which "
                "is not part of this build: launches always run the CUDA kernels.")
        if num_warps not in (1, 2, 4, 8, 16, 32):
            raise ValueError(f"num_warps must be a power of two from 1 to 32, but got {num_warps}")
        if dot_backend not in ("auto", "simdgroup", "mpp"):
            raise ValueError(f"dot_backend must be 'auto', 'simdgroup', or 'mpp', not {dot_backend!r}")
        names = self.arg_names
        if len(args) + len(kwargs) == len(names) and len(args) <= len(names):
            # fast path: every parameter given once (positional prefix + keywords), no defaults needed
            bound = dict(zip(names, args))
            bound.update(kwargs)
            if len(bound) != len(names) or any(n not in bound for n in names[len(args):]):
                bound = self.bind(args, kwargs)
        else:
            bound = self.bind(args, kwargs)
        for n in self._constexpr_names:
            v = bound[n]
            if isinstance(v, tl.constexpr):
                bound[n] = v.value
        g = resolve_grid(grid, bound)
        if g[0] == 0 or g[1] == 0 or g[2] == 0:
            return  # src/enceladus/runtime/launcher.py:459-460
        ad = self.adapter()
        v = self.variant if variant is None else variant
        launch(ad, bound, g, -1 if v is None else int(v), self)

    def warmup(self, *args: Any, grid: Any = None, num_warps: int = 4, dot_warps: tuple[int, int] | None = None,
               dot_backend: str = "auto", variant: int | None = None, **kwargs: Any) -> CompiledKernel:
        """Does everything a launch does short of launching: binds the arguments, finds the native kernel and
        loads the library (src/enceladus/runtime/jit.py:527-537 compiles without launching; here the kernels
        are compiled ahead of time, so the costs that remain are the library load and the symbol lookup).

        Raises what a launch would raise for an unknown kernel, a bad binding or a missing library.
        """
        if num_warps not in (1, 2, 4, 8, 16, 32):
            raise ValueError(f"num_warps must be a power of two from 1 to 32, but got {num_warps}")
        self.bind(args, kwargs)
        ad = self.adapter()
        n = N.num_variants(ad.kernel_id)
        v = self.variant if variant is None else variant
        v = -1 if v is None else int(v)
        if v >= n:
            raise ValueError(f"{self.__name__}: variant {v} is out of range, the kernel has {n}")
        return CompiledKernel(self.__name__, _ENTRY_POINTS[ad.kernel_id],
                              tuple(N.variant_info(ad.kernel_id, i) for i in range(n)), v, num_warps)

    def explain(self, *args: Any, grid: Any = None, num_warps: int = 4, dot_warps: tuple[int, int] | None = None,
                dot_backend: str = "auto", variant: int | None = None, **kwargs: Any) -> str:
        """Prints and returns what a launch with these arguments would run.

        The reference reports tile layouts, register estimates and threadgroup memory of the code it
        generates (src/enceladus/runtime/jit.py:539-573).  Nothing is generated here; the report names the
        native entry point, the array arguments with their dtypes and shapes, and the tile variants with the
        one in force.
        """
        ck = self.warmup(*args, num_warps=num_warps, dot_warps=dot_warps, dot_backend=dot_backend, variant=variant,
                         **kwargs)
        bound = self.bind(args, kwargs)
        ad = self.adapter()
        lines = [f"kernel {self.__name__} -> {ck.entry} (libenc_b200.so, precompiled for sm_100a)"]
        if grid is not None:
            lines.append(f"  grid {resolve_grid(grid, {k: (v.value if isinstance(v, tl.constexpr) else v) for k, v in bound.items()})}")
        for name in ad.array_list:
            a = bound[name]
            role = "out" if name in ad.outputs else "in"
            lines.append(f"  {role:3s} {name}: {getattr(a, 'dtype', type(a).__name__)} {tuple(getattr(a, 'shape', ()))}")
        consts = {n: bound[n] for n in self._constexpr_names}
        if consts:
            lines.append("  constexpr " + ", ".join(f"{k}={v.value if isinstance(v, tl.constexpr) else v}" for k, v in consts.items()))
        lines.append("  num_warps / dot_warps / dot_backend describe Apple SIMD-group layouts and are ignored")
        for i, info in enumerate(ck.variants):
            mark = "*" if i == ck.variant else " "
            lines.append(f"  {mark} variant {i}: {info}")
        if ck.variant < 0:
            lines.append("  variant in force: chosen by the library from the shape")
        text = "\n".join(lines)
        print(text)
        return text


@dataclass(frozen=True)
class CompiledKernel:
    """What `JITFunction.warmup` returns: the precompiled native kernel a launch with these arguments uses.

    The reference's object of the same name carries the generated MSL and IR
    (src/enceladus/runtime/jit.py:527-537); nothing is generated here, so it names the native entry point
    and lists the hand-written tile variants instead.
    """

    name: str
    entry: str
    variants: tuple[str, ...]
    variant: int  # -1: the library chooses per shape
    num_warps: int


_ENTRY_POINTS = {N.K_SOFTMAX: "enc_softmax", N.K_LAYERNORM: "enc_layernorm", N.K_RMSNORM: "enc_rmsnorm",
                 N.K_GELU: "enc_gelu", N.K_MATMUL: "enc_matmul", N.K_ATTENTION: "enc_attention_fwd",
                 N.K_HISTOGRAM: "enc_histogram", N.K_CUMSUM: "enc_cumsum", N.K_ADD: "enc_add",
                 N.K_MATMUL_INT: "enc_matmul_int"}


def launch(ad, bound: dict[str, Any], grid: tuple[int, int, int], variant: int, jf: JITFunction | None) -> None:
    """Resolves array arguments to device memory, calls the adapter, writes NumPy outputs back."""
    tensor = interop.tensor_type()
    dev = None
    host_names = None
    for name in ad.array_list:
        v = bound[name]
        if isinstance(v, tensor):
            if not v.is_cuda:
                raise TypeError(f"argument `{name}` is a torch tensor on {v.device}; pass a CUDA tensor "
                                "or a NumPy array")
            if dev is None:
                dev, dev_name = v.device, name
            elif v.device != dev:
                # a pointer into another GPU's memory would reach the kernel as a peer (or foreign) address
                raise ValueError(f"argument `{name}` lives on {v.device} but `{dev_name}` lives on {dev}; "
                                 "all array arguments of one launch must be on the same device")
        elif isinstance(v, np.ndarray):
            host_names = [name] if host_names is None else [*host_names, name]
        else:
            raise TypeError(f"argument `{name}` must be a NumPy array or a torch CUDA tensor, not "
                            f"{type(v).__name__}")
    torch = interop._torch()
    if host_names is None:  # hot path: every array already lives on the device
        if dev.index != torch.cuda.current_device():
            with torch.cuda.device(dev):
                ad.fn(bound, grid, variant, interop.current_stream())
        else:
            ad.fn(bound, grid, variant, interop.current_stream())
        return
    if dev is not None and dev.index != torch.cuda.current_device():
        raise ValueError("NumPy arguments are staged on the current CUDA device, but the tensor arguments "
                         f"live on {dev}; make it current with torch.cuda.set_device first")
    if ad.split is not None and not interop.async_numpy_enabled():
        plan = _pipeline_plan(ad, bound, grid, host_names)
        if plan is not None:
            _launch_pipelined(ad, bound, grid, variant, jf, host_names, *plan)
            return
    staged = interop.Staged()
    resolved = dict(bound)
    extents = ad.extents(bound, grid) if ad.extents is not None else {}
    for name in host_names:
        v = bound[name]
        dense = v.flags.c_contiguous and extents.get(name) == v.size
        resolved[name] = staged.to_device(name, v, name in ad.outputs, overwritten=dense)
    ad.fn(resolved, grid, variant, interop.current_stream())
    staged.finish()
    if jf is not None:
        jf.last_launch = {"h2d_bytes": staged.h2d_bytes, "d2h_bytes": staged.d2h_bytes, "variant": variant}


PIPELINE_MIN_BYTES = 16 << 20   # below this much partitioned host data a launch is staged in one piece
PIPELINE_PIECE_BYTES = 32 << 20  # target size of a piece, inputs and outputs together (measured best of 16-128 MB)
PIPELINE_STREAMS = 2  # one per direction of the link
_side_streams: dict[int, list[Any]] = {}


def _pipeline_plan(ad, bound: dict[str, Any], grid: tuple[int, int, int], host_names: list[str]):
    """Decides whether a launch with NumPy arguments is staged piecewise; returns (split, pieces) or None.

    Every partitioned array must be a C-contiguous NumPy array (its flat view is then a view), every piece
    must start on a 256-byte boundary in every array (the kernels' vector paths need 16), and there must be
    enough data for the overlap to pay for the extra launches.
    """
    sp = ad.split(bound, grid)
    if sp is None or sp.units < 2:
        return None
    total = 0
    align = 1  # pieces start at multiples of this many units
    for name, per in sp.arrays.items():
        v = bound[name]
        if not isinstance(v, np.ndarray) or not v.flags.c_contiguous or per <= 0:
            return None
        total += min(v.size, sp.units * per) * v.itemsize
        step = per * v.itemsize
        need = 256 // np.gcd(256, step)
        align = align * need // np.gcd(align, need)
    if any(n not in sp.arrays and isinstance(bound[n], np.ndarray) and n in ad.outputs for n in host_names):
        return None  # a shared output would be written by every piece
    if total < PIPELINE_MIN_BYTES:
        return None
    pieces = int(max(2, min(32, total // PIPELINE_PIECE_BYTES)))
    per_piece = -(-sp.units // pieces)
    per_piece = int(-(-per_piece // align) * align)  # (align is a NumPy integer)
    if per_piece >= sp.units:
        return None
    return sp, [(u0, min(per_piece, sp.units - u0)) for u0 in range(0, sp.units, per_piece)]


def _launch_pipelined(ad, bound, grid, variant, jf, host_names, sp, pieces) -> None:
    """Stages, runs and copies back one piece after the other, then waits for all of it: the launch is complete
    when this returns, as the one-piece path is.

    Two side streams, one per direction of the link: copies in and the kernels on the first, copies out on the
    second, an event per piece between them.  Copies of one direction then run one after the other in piece
    order, so the first piece's kernel starts after one piece's transfer and the link is busy both ways from
    then on.  (Measured on B200, LayerNorm bf16 [16384, 4096] from pinned memory: 3.13 ms against 3.68 ms with
    whole pieces dealt round-robin to three streams, where the copies in of neighbouring pieces shared the
    link and every kernel started late; smaller pieces at both ends of the schedule did not pay, each extra
    piece costs about 50 us.)"""
    torch = interop._torch()
    cur = torch.cuda.current_stream()
    di = torch.cuda.current_device()
    streams = _side_streams.get(di)
    if streams is None:
        streams = _side_streams[di] = [torch.cuda.Stream() for _ in range(PIPELINE_STREAMS)]
    s_in, s_out = streams
    staged = interop.Staged()
    shared = dict(bound)
    ready = cur.record_event()
    s_in.wait_event(ready)
    s_out.wait_event(ready)
    extents = ad.extents(bound, grid) if ad.extents is not None else {}
    flat = {name: bound[name].reshape(-1) for name in sp.arrays}
    dense = {name: extents.get(name) == bound[name].size for name in sp.arrays}
    # An output in pageable host memory cannot be copied out piece by piece: such a copy blocks the host until
    # the stream gets there.  It is staged whole, the pieces write slices of it, and one copy follows at the end.
    whole: dict[str, Any] = {}
    try:
        with torch.cuda.stream(s_in):
            for name in host_names:
                if name not in sp.arrays:
                    shared[name] = staged.to_device(name, bound[name], False)
            for name in sp.arrays:
                if name in ad.outputs and not interop._np_as_torch_view(flat[name]).is_pinned():
                    whole[name] = staged.to_device(name, flat[name], True, overwritten=dense[name])
        before = None
        for u0, n in pieces:
            with torch.cuda.stream(s_in):
                piece = dict(shared)
                piece.update(sp.rebind(n))
                views = []
                for name, per in sp.arrays.items():
                    lo, hi = u0 * per, min((u0 + n) * per, flat[name].size)
                    if name in whole:
                        piece[name] = whole[name][lo:hi]
                        continue
                    host = flat[name][lo:hi]
                    written = name in ad.outputs
                    piece[name] = staged.to_device(name, host, written, overwritten=dense[name])
                    if written:
                        piece[name].record_stream(s_out)  # allocated on s_in, read by the copy out on s_out
                        views.append((piece[name], host))
                if sp.chain is not None:
                    sp.chain(piece, before)
                    before = piece
                ad.fn(piece, sp.grid(n), variant, int(s_in.cuda_stream))
                done = s_in.record_event()
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for d, host in views:
                    interop._np_as_torch_view(host).copy_(d, non_blocking=True)
                    staged.d2h_bytes += host.nbytes
    finally:
        for st in streams:
            st.synchronize()
    for name, d in whole.items():
        interop._np_as_torch_view(flat[name]).copy_(d)
        staged.d2h_bytes += flat[name].nbytes
    staged.writeback.clear()
    if jf is not None:
        jf.last_launch = {"h2d_bytes": staged.h2d_bytes, "d2h_bytes": staged.d2h_bytes, "variant": variant,
                          "pieces": len(pieces)}


def jit(fn: Callable[..., Any] | None = None, *, interpret: bool | None = None,
        do_not_specialize: Iterable[str | int] = (), math_mode: str = "relaxed"):
    """Decorator that turns a kernel definition into a launchable `JITFunction` (jit.py:1237-1264)."""
    if fn is not None:
        return JITFunction(fn, interpret=interpret, do_not_specialize=do_not_specialize, math_mode=math_mode)
    return lambda f: JITFunction(f, interpret=interpret, do_not_specialize=do_not_specialize,
                                 math_mode=math_mode)
