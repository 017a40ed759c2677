"""ctypes binding of libenc_b200.so (declared in include/enceladus_b200.h).

This is the counterpart of the reference's nanobind module `enceladus._C`
(src/enceladus/_C/bindings.mm): the only place where Python meets the native library.  There is no
CPU fallback: if the library is missing or cannot be loaded, every launch raises `CudaError`.
ctypes releases the GIL for the duration of each call, as the reference does around sync and
compile (bindings.mm:513,593).
"""

from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libenc_b200.so"

# enc_status
OK, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_LAUNCH, ERR_DEVICE_WAIT, ERR_NO_MEMORY = range(6)
# enc_dtype
F32, F16, BF16, I32, I8, I16, I64, U8 = range(8)
# enc_kernel
K_SOFTMAX, K_LAYERNORM, K_RMSNORM, K_GELU, K_MATMUL, K_ATTENTION, K_HISTOGRAM, K_CUMSUM, K_ADD, K_MATMUL_INT = range(10)
VARIANT_AUTO = -1


class CudaError(RuntimeError):
    """A failure reported by the native library or by CUDA.

    Plays the role of `enceladus.MetalError` (src/enceladus/_C/bindings.mm:21-23,341): GPU-side errors
    surface at the launch that detects them or at the next `synchronize()`.
    """

    def __init__(self, message: str, status: int = ERR_LAUNCH) -> None:
        super().__init__(message)
        self.status = status


class DeviceInfo(C.Structure):
    _fields_ = [("device", C.c_int), ("sm_count", C.c_int), ("cc_major", C.c_int),
                ("cc_minor", C.c_int), ("max_smem_per_block", C.c_int), ("l2_bytes", C.c_int),
                ("global_mem", C.c_uint64), ("name", C.c_char * 128)]


_p, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float

# name -> argtypes; every function returns int unless listed in _RESTYPES
SIGNATURES: dict[str, list] = {
    "enc_last_error": [],
    "enc_device_info": [C.POINTER(DeviceInfo)],
    "enc_num_variants": [_i],
    "enc_variant_info": [_i, _i, C.c_char_p, C.c_size_t],
    "enc_synchronize": [_p],
    "enc_softmax": [_p, _p, _i64, _i64, _i64, _i64, _i, _i, _p],
    "enc_layernorm": [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _f, _i, _i, _p],
    "enc_rmsnorm": [_p, _p, _p, _i64, _i64, _i64, _i64, _f, _i, _i, _p],
    "enc_gelu": [_p, _p, _p, _i64, _i64, _f, _i, _i, _i, _i, _p],
    "enc_add": [_p, _p, _p, _i64, _i, _i, _p],
    "enc_histogram": [_p, _p, _i64, _f, _f, _i64, _i, _i, _p],
    "enc_cumsum": [_p, _p, _i64, _i64, _i64, _i64, _i, _i, _p, _i, _p],
    "enc_cumsum_noalloc": [_p, _p, _i64, _i, _p, _p, _p],
    "enc_cumsum_out_dtype": [_i],
    "enc_sum": [_p, _p, _i64, _i, _p],
    "enc_scan_offset": [_p, _i, _i, _p, _i, _p],
    "enc_matmul": [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _p],
    "enc_matmul_int": [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i, _i, _p],
    "enc_attention_fwd": [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _f, _i, _i, _i, _p],
    "enc_test_fail_next": [_i],
    "enc_test_device_wait": [C.c_uint, _p],
}
_RESTYPES = {"enc_last_error": C.c_char_p, "enc_test_fail_next": None}

_lib = None
_lock = threading.Lock()


def load() -> C.CDLL:
    """Loads the library once and declares every prototype.  Raises `CudaError` if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = Path(os.environ.get("ENCELADUS_B200_LIB", LIB_PATH))
        if not path.exists():
            raise CudaError(
                f"the CUDA kernel library {path} is not built. Run `python -m enceladus_b200.build` "
                "(needs nvcc). There is no CPU fallback.")
        try:
            lib = C.CDLL(str(path))
        except OSError as e:
            raise CudaError(f"cannot load {path}: {e}") from None
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here means header and library disagree
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(name, C.c_int)
        _lib = lib
    return _lib


def is_loaded() -> bool:
    return _lib is not None


def last_error() -> str:
    return load().enc_last_error().decode("utf-8", "replace")


_EXC = {ERR_BAD_ARG: ValueError, ERR_UNSUPPORTED: NotImplementedError}


def check(status: int) -> None:
    """Raises the Python exception that corresponds to a non-zero enc_status."""
    if status == OK:
        return
    msg = last_error() or f"enc_status {status}"
    exc = _EXC.get(status)
    if exc is not None:
        raise exc(msg)
    raise CudaError(msg, status)


def call(name: str, *args) -> None:
    check(getattr(load(), name)(*args))


def device_info() -> DeviceInfo:
    info = DeviceInfo()
    call("enc_device_info", C.byref(info))
    return info


def num_variants(kernel: int) -> int:
    return load().enc_num_variants(kernel)


def variant_info(kernel: int, variant: int) -> str:
    buf = C.create_string_buffer(256)
    call("enc_variant_info", kernel, variant, buf, len(buf))
    return buf.value.decode()
