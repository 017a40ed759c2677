"""The `tl` namespace that kernel definitions import: `import enceladus_b200.language as tl`.

Kernels in this build are hand-written CUDA; a `@jit` function's Python body is documentation of what
the native kernel computes and is never executed.  The namespace therefore only has to make kernel
modules importable: `tl.constexpr` for parameter annotations, the dtype objects, and the builtin
names, which raise when called outside a kernel exactly as the reference's do
(src/enceladus/language/core.py:306-312).
"""

from __future__ import annotations

from typing import Any

import numpy as np


class dtype:  # noqa: N801 - mirrors `enceladus.language.dtype`
    """An element type (src/enceladus/language/core.py:105-121)."""

    def __init__(self, name: str, kind: str, bits: int, long_name: str) -> None:
        self.name, self.kind, self.primitive_bitwidth, self.long_name = name, kind, bits, long_name

    def __repr__(self) -> str:
        return f"tl.{self.long_name}"

    def is_floating(self) -> bool:
        return self.kind == "float"

    def is_int(self) -> bool:
        return self.kind in ("int", "uint", "bool")

    def to_numpy(self) -> np.dtype:
        if self.long_name == "bfloat16":
            import ml_dtypes

            return np.dtype(ml_dtypes.bfloat16)
        return np.dtype("bool" if self.long_name == "int1" else self.long_name)


int1 = dtype("i1", "bool", 1, "int1")
int8 = dtype("i8", "int", 8, "int8")
int16 = dtype("i16", "int", 16, "int16")
int32 = dtype("i32", "int", 32, "int32")
int64 = dtype("i64", "int", 64, "int64")
uint8 = dtype("u8", "uint", 8, "uint8")
uint16 = dtype("u16", "uint", 16, "uint16")
uint32 = dtype("u32", "uint", 32, "uint32")
uint64 = dtype("u64", "uint", 64, "uint64")
float16 = dtype("fp16", "float", 16, "float16")
bfloat16 = dtype("bf16", "float", 16, "bfloat16")
float32 = dtype("fp32", "float", 32, "float32")


class constexpr:  # noqa: N801 - matches `triton.language.constexpr`
    """Marks a kernel parameter as a compile-time constant, or wraps a constant value
    (src/enceladus/language/core.py:193-228)."""

    __slots__ = ("value",)

    def __init__(self, value: Any) -> None:
        self.value = value.value if isinstance(value, constexpr) else value

    def __repr__(self) -> str:
        return f"constexpr({self.value!r})"

    def __eq__(self, other: object) -> bool:
        return unwrap(self) == unwrap(other)

    def __hash__(self) -> int:
        return hash(self.value)

    def __bool__(self) -> bool:
        return bool(self.value)

    def __index__(self) -> int:
        return self.value.__index__()

    def __int__(self) -> int:
        return int(self.value)

    def __float__(self) -> float:
        return float(self.value)


def unwrap(value: Any) -> Any:
    return value.value if isinstance(value, constexpr) else value


def is_constexpr_annotation(ann: Any) -> bool:
    if ann is constexpr or isinstance(ann, constexpr):
        return True
    return isinstance(ann, str) and ann.replace(" ", "").split(".")[-1] == "constexpr"


class _Builtin:
    def __init__(self, name: str) -> None:
        self.__name__ = name

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        raise RuntimeError(
            f"tl.{self.__name__} can only be called inside a @jit kernel, and this build does not "
            "execute kernel bodies in Python: launches go to hand-written CUDA kernels.")

    def __repr__(self) -> str:
        return f"<tl.{self.__name__}>"


_BUILTINS = (
    "abs arange argmax argmin associative_scan atomic_add atomic_and atomic_cas atomic_max atomic_min "
    "atomic_or atomic_xchg atomic_xor broadcast_to cast cdiv ceil clamp cos cumsum debug_barrier "
    "device_assert device_print dot erf exp exp2 expand_dims floor fma full full_like join load log "
    "log2 make_tensor_descriptor max max_contiguous maximum min minimum multiple_of num_programs "
    "permute program_id range reduce reshape rsqrt sigmoid sin split sqrt static_assert static_print "
    "static_range store sum tanh trans where zeros zeros_like"
).split()
for _n in _BUILTINS:
    globals()[_n] = _Builtin(_n)
del _n

__all__ = ["constexpr", "dtype", "int1", "int8", "int16", "int32", "int64", "uint8", "uint16",
           "uint32", "uint64", "float16", "bfloat16", "float32", *_BUILTINS]
