"""Candidate configurations for the autotuner (counterpart of src/enceladus/configs.py).

The reference lists (BM, BN, BK, num_warps, dot_warps) shapes measured on Apple GPUs.  Here each
candidate names one hand-written tile variant of the CUDA kernel; `BM`/`BN`/`BK` (or
`BLOCK_M`/`BLOCK_N`) are the tile the variant really uses, so a launch grid computed from them covers
the problem.
"""

from __future__ import annotations

from typing import Any

import numpy as np

from enceladus_b200.runtime.autotuner import Config

_FP32_NAMES = ("float32", "fp32", "f32")
_HALF_NAMES = ("float16", "fp16", "f16", "half", "bfloat16", "bf16")

# (BM, BN, BK, stages) of the tcgen05 matmul variants, in the order the native library numbers them.
MATMUL_TILES = [(128, 256, 64, 4), (128, 128, 64, 6), (128, 256, 64, 3), (128, 64, 64, 8)]
# (BLOCK_M, BLOCK_N) of the attention variants.
ATTENTION_TILES = [(256, 128), (128, 128), (128, 128), (256, 64), (256, 64)]


def _dtype_name(dtype: Any) -> str:
    if isinstance(dtype, str):
        name = dtype
    elif hasattr(dtype, "long_name"):
        name = dtype.long_name
    else:
        try:
            name = np.dtype(dtype).name
        except (TypeError, ValueError):
            name = str(dtype)
    return name.rsplit(".", 1)[-1]


def matmul_configs(dtype: Any = "float16") -> list[Config]:
    """The matmul configurations to autotune over for `dtype` (float16 or bfloat16 on tensor cores).

    Raises:
        ValueError: `dtype` isn't float32, float16, or bfloat16.
    """
    name = _dtype_name(dtype)
    if name not in _FP32_NAMES + _HALF_NAMES:
        raise ValueError(f"matmul_configs supports float32, float16, and bfloat16, but got {name}. "
                         "Pass the dtype of the matmul operands.")
    return [Config({"BM": bm, "BN": bn, "BK": bk}, num_warps=4, variant=i)
            for i, (bm, bn, bk, _) in enumerate(MATMUL_TILES)]


def attention_configs(dtype: Any = "float16", head_dim: int = 64) -> list[Config]:
    """The flash-attention configurations to autotune over.

    Raises:
        ValueError: `dtype` or `head_dim` isn't supported.
    """
    name = _dtype_name(dtype)
    if name not in _FP32_NAMES + _HALF_NAMES:
        raise ValueError(f"attention_configs supports float32, float16, and bfloat16, but got {name}. "
                         "Pass the dtype of q, k, and v.")
    if head_dim not in (16, 32, 64, 128):
        raise ValueError(f"attention_configs supports head dimensions 16, 32, 64, and 128, but got {head_dim}")
    return [Config({"BLOCK_M": bm, "BLOCK_N": bn}, num_warps=4, dot_warps=(4, 1), variant=i)
            for i, (bm, bn) in enumerate(ATTENTION_TILES)]
