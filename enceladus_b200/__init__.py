"""enceladus_b200: the Enceladus kernel set as hand-written CUDA for NVIDIA B200 (sm_100a).

Use it the way the reference package is used (src/enceladus/__init__.py:12-45):

    import enceladus_b200 as enceladus
    import enceladus_b200.language as tl

`@enceladus.jit` kernels are launched as `kernel[grid](...)` with torch CUDA tensors or NumPy arrays;
the launch is routed to the matching kernel in libenc_b200.so.  The host wrappers of the kernel set
(`softmax`, `layernorm`, `rmsnorm`, `fused_gelu`, `matmul_bias_gelu`, `attention`, `histogram`, `cumsum`,
...) live in `enceladus_b200.ops`.
"""

from enceladus_b200 import language
from enceladus_b200._native import CudaError
from enceladus_b200.language import constexpr
from enceladus_b200.runtime.autotuner import Config, autotune, heuristics
from enceladus_b200.runtime.interop import (
    async_numpy,
    element_dtype,
    element_strides,
    new_empty,
    new_zeros,
    synchronize,
)
from enceladus_b200.runtime.jit import JITFunction, cdiv, jit, next_power_of_2

__version__ = "0.1.0"

# The reference's name for a GPU-side failure; kept so that `except enceladus.MetalError` still works.
MetalError = CudaError

_LAZY_SUBMODULES = ("configs", "testing", "ops", "dist", "workloads")


def __getattr__(name: str):
    if name in _LAZY_SUBMODULES:
        import importlib

        return importlib.import_module(f"enceladus_b200.{name}")
    raise AttributeError(f"module 'enceladus_b200' has no attribute {name!r}")


def __dir__() -> list[str]:
    return sorted([*globals(), *_LAZY_SUBMODULES])
