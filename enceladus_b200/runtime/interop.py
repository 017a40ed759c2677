"""Array arguments: torch CUDA tensors (zero-copy) and NumPy host arrays (staged through the device).

Replaces the reference's interop layer (src/enceladus/runtime/interop.py), whose array kinds are
`enceladus.Tensor` (Metal shared memory), torch-mps tensors and MLX arrays.  Here:

  * a torch CUDA tensor is passed by `data_ptr()`; the launch is enqueued on torch's current CUDA
    stream, so it is ordered with the surrounding torch ops without a sync (the reference launches on
    PyTorch's own MPS stream for the same effect, src/enceladus/runtime/launcher.py:106-200);
  * a NumPy array is copied to the device before the launch and, if the kernel writes it, copied back
    after — the reference's copy-in/write-back fallback (interop.py:563-574).  The results are in the
    array when the launch returns, unless `async_numpy(True)`, in which case after `synchronize()`.
"""

from __future__ import annotations

import contextlib
import threading
from typing import Any

import numpy as np

from enceladus_b200 import _native as N

try:
    import ml_dtypes

    BF16 = np.dtype(ml_dtypes.bfloat16)
except ImportError:  # pragma: no cover
    BF16 = None

_NP_CODES = {np.dtype(np.float32): N.F32, np.dtype(np.float16): N.F16, np.dtype(np.int32): N.I32,
             np.dtype(np.int8): N.I8, np.dtype(np.int16): N.I16, np.dtype(np.int64): N.I64,
             np.dtype(np.uint8): N.U8}
if BF16 is not None:
    _NP_CODES[BF16] = N.BF16

_state = threading.local()
_pending: list[tuple[Any, np.ndarray]] = []  # (device tensor, host array) awaiting write-back
_pending_lock = threading.Lock()


_torch_mod = None
_TORCH_NP: dict[Any, np.dtype] = {}   # torch dtype -> NumPy dtype
_TORCH_CODE: dict[Any, int] = {}      # torch dtype -> enc_dtype


def _torch():
    """torch, imported on first use (importing it costs seconds), with the dtype tables filled."""
    global _torch_mod
    if _torch_mod is None:
        import torch

        _TORCH_NP.update({torch.float32: np.dtype(np.float32), torch.float16: np.dtype(np.float16),
                          torch.bfloat16: BF16, torch.int32: np.dtype(np.int32), torch.int8: np.dtype(np.int8),
                          torch.int16: np.dtype(np.int16), torch.int64: np.dtype(np.int64),
                          torch.uint8: np.dtype(np.uint8), torch.bool: np.dtype(np.bool_)})
        _TORCH_CODE.update({t: _NP_CODES[d] for t, d in _TORCH_NP.items() if d in _NP_CODES})
        _torch_mod = torch
    return _torch_mod


def tensor_type():
    return _torch().Tensor


def is_torch(obj: Any) -> bool:
    return isinstance(obj, _torch().Tensor)


def is_array(obj: Any) -> bool:
    return isinstance(obj, np.ndarray) or is_torch(obj)


def _torch_np_dtype(t: Any) -> np.dtype:
    _torch()
    try:
        return _TORCH_NP[t.dtype]
    except KeyError:
        raise TypeError(f"torch dtype {t.dtype} isn't supported by enceladus_b200") from None


def _np_to_torch_dtype(dt: Any):
    torch = _torch()
    dt = np.dtype(dt)
    if BF16 is not None and dt == BF16:
        return torch.bfloat16
    return {np.dtype(np.float32): torch.float32, np.dtype(np.float16): torch.float16,
            np.dtype(np.int32): torch.int32, np.dtype(np.int8): torch.int8,
            np.dtype(np.int16): torch.int16, np.dtype(np.int64): torch.int64,
            np.dtype(np.uint8): torch.uint8, np.dtype(np.bool_): torch.bool}[dt]


_UNSUPPORTED = ("{} isn't a supported array type. Pass a NumPy array or a torch tensor on a CUDA "
                "device.")


def element_strides(obj: Any) -> tuple[int, ...]:
    """Strides of a supported array, in elements (src/enceladus/runtime/interop.py:323-345)."""
    if isinstance(obj, np.ndarray):
        return tuple(s // obj.itemsize for s in obj.strides)
    if is_torch(obj):
        return tuple(obj.stride())
    raise TypeError(_UNSUPPORTED.format(type(obj).__name__))


def element_dtype(obj: Any) -> np.dtype:
    """Element type of a supported array as a NumPy dtype (interop.py:348-365)."""
    if isinstance(obj, np.ndarray):
        return obj.dtype
    if is_torch(obj):
        return _torch_np_dtype(obj)
    raise TypeError(_UNSUPPORTED.format(type(obj).__name__))


def dtype_code(obj: Any) -> int:
    if not isinstance(obj, np.ndarray):
        code = _TORCH_CODE.get(getattr(obj, "dtype", None))
        if code is not None:
            return code
    dt = element_dtype(obj)
    try:
        return _NP_CODES[dt]
    except KeyError:
        raise TypeError(f"element type {dt} isn't supported by the CUDA kernels") from None


def _new_array(like: Any, shape: Any, dtype: Any, zero: bool) -> Any:
    shape = tuple(like.shape) if shape is None else tuple(shape)
    if isinstance(like, np.ndarray):
        dt = np.dtype(like.dtype if dtype is None else dtype)
        big = int(np.prod(shape)) * dt.itemsize >= PINNED_MIN_BYTES
        if big and not zero and (dt in _NP_CODES) and _torch().cuda.is_available():
            return _pinned_empty(shape, dt)
        return (np.zeros if zero else np.empty)(shape, dt)
    if is_torch(like):
        torch = _torch()
        td = like.dtype if dtype is None else (dtype if isinstance(dtype, torch.dtype) else _np_to_torch_dtype(dtype))
        return (torch.zeros if zero else torch.empty)(shape, dtype=td, device=like.device)
    raise TypeError(_UNSUPPORTED.format(type(like).__name__))


PINNED_MIN_BYTES = 1 << 20


def _pinned_empty(shape: tuple[int, ...], dt: np.dtype) -> np.ndarray:
    """An uninitialised NumPy array in page-locked host memory.

    Large NumPy outputs are copied back from the device; page-locked memory makes that copy run at
    full PCIe speed and avoids first-touch page faults.  The block comes from torch's caching host
    allocator, so repeated launches of one shape reuse it; the array keeps the block alive.
    """
    torch = _torch()
    if BF16 is not None and dt == BF16:
        return torch.empty(shape, dtype=torch.uint16, pin_memory=True).numpy().view(BF16)
    return torch.empty(shape, dtype=_np_to_torch_dtype(dt), pin_memory=True).numpy()


def new_empty(like: Any, shape: Any = None, dtype: Any = None) -> Any:
    """An uninitialised array of the same kind and device as `like` (interop.py:393-412)."""
    return _new_array(like, shape, dtype, zero=False)


def new_zeros(like: Any, shape: Any = None, dtype: Any = None) -> Any:
    """A zero-filled array of the same kind and device as `like` (interop.py:415-420)."""
    return _new_array(like, shape, dtype, zero=True)


@contextlib.contextmanager
def _async_ctx(prev: bool):
    try:
        yield
    finally:
        _state.async_numpy = prev


def async_numpy(enabled: bool = True):
    """Lets launches with NumPy arguments return before their results are copied back.

    With it on, outputs land in the NumPy arrays at the next `synchronize()`.  Usable as a plain call
    or as a context manager (src/enceladus/runtime/interop.py:495-503).
    """
    prev = getattr(_state, "async_numpy", False)
    _state.async_numpy = bool(enabled)
    return _async_ctx(prev)


def async_numpy_enabled() -> bool:
    return getattr(_state, "async_numpy", False)


def current_stream() -> int:
    return int(_torch().cuda.current_stream().cuda_stream)


def _np_as_torch_view(a: np.ndarray):
    """A torch CPU tensor sharing the memory of a NumPy array (bfloat16 through its uint16 bits)."""
    torch = _torch()
    if BF16 is not None and a.dtype == BF16:
        return torch.from_numpy(a.view(np.uint16)).view(torch.bfloat16)
    if a.dtype == np.bool_:
        return torch.from_numpy(a.view(np.uint8))
    return torch.from_numpy(a)


class Staged:
    """Device copies of the NumPy arguments of one launch."""

    def __init__(self) -> None:
        self.writeback: list[tuple[Any, np.ndarray]] = []
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def to_device(self, name: str, a: np.ndarray, written: bool, overwritten: bool = False):
        torch = _torch()
        if not torch.cuda.is_available():
            raise N.CudaError("no CUDA device is available, and there is no CPU fallback")
        if written and not a.flags.writeable:
            raise ValueError(f"argument `{name}` is a read-only NumPy array, but the kernel writes it")
        if any(s < 0 for s in a.strides):
            raise ValueError(f"argument `{name}` has a negative stride, which kernels can't address")
        if not a.flags.c_contiguous and a.size:
            # A view with strided rows or other gaps: the kernel addresses it with the host strides, so the
            # device copy must keep them.  Stage the whole span from the first to the last element.
            span = sum((n - 1) * st for n, st in zip(a.shape, a.strides)) // a.itemsize + 1
            a = np.lib.stride_tricks.as_strided(a, shape=(span,), strides=(a.itemsize,), writeable=a.flags.writeable)
            overwritten = False
        host = _np_as_torch_view(a)
        if written and overwritten:
            dev = torch.empty_like(host, device="cuda")  # every element is produced by the kernel
        else:
            # Partly written outputs are copied in as well (masked stores, strided rows, accumulating
            # atomics): the write-back must preserve what the kernel does not touch.
            dev = host.to("cuda", non_blocking=True)
            self.h2d_bytes += a.nbytes
        if written:
            self.writeback.append((dev, a))
        return dev

    def finish(self) -> None:
        """Copies written arrays back; waits unless async_numpy is on."""
        if not self.writeback:
            return
        if async_numpy_enabled():
            with _pending_lock:
                _pending.extend(self.writeback)
            return
        for dev, a in self.writeback:
            _np_as_torch_view(a).copy_(dev)  # synchronous D2H on the current stream
            self.d2h_bytes += a.nbytes


def flush_pending() -> None:
    with _pending_lock:
        items, _pending[:] = list(_pending), []
    for dev, a in items:
        _np_as_torch_view(a).copy_(dev)


def synchronize() -> None:
    """Waits for all launched work and raises `CudaError` for any GPU-side failure since the last
    synchronisation (replaces src/enceladus/runtime/stream.py synchronize)."""
    torch = _torch()
    if not torch.cuda.is_available():
        raise N.CudaError("no CUDA device is available")
    N.call("enc_synchronize", current_stream())
    flush_pending()
