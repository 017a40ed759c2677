"""The C-ABI library loads and exports every symbol that include/enceladus_b200.h declares.

No compute calls here (no GPU needed): symbols, prototypes, argument validation that happens before
any CUDA call, the status/message plumbing and the host-side failure hook.
"""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

from enceladus_b200 import _native as N

ROOT = Path(__file__).resolve().parents[1]
HEADER = (ROOT / "include" / "enceladus_b200.h").read_text()


@pytest.fixture(scope="module")
def lib():
    from enceladus_b200 import build

    build.build()
    return N.load()


def declared_functions() -> list[str]:
    code = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    return sorted(set(re.findall(r"\b(enc_[a-z0-9_]+)\s*\(", code)))


def test_header_declares_what_the_binding_binds():
    assert declared_functions() == sorted(N.SIGNATURES)


def test_every_declared_symbol_is_exported(lib):
    raw = ctypes.CDLL(str(N.LIB_PATH))
    for name in declared_functions():
        assert hasattr(raw, name), f"{name} is declared in the header but not exported"


def test_every_entry_point_cites_the_reference_interface():
    # each kernel entry point names the reference kernel or runtime call it replaces
    for name in ("enc_softmax", "enc_layernorm", "enc_rmsnorm", "enc_gelu", "enc_add", "enc_histogram",
                 "enc_cumsum", "enc_matmul", "enc_attention_fwd", "enc_synchronize", "enc_device_info"):
        before = HEADER[: HEADER.index(f" {name}(")]
        comment = before[before.rindex("/*"):]
        assert re.search(r"(examples/|src/enceladus/|enceladus_rt\.h)", comment), name


def test_status_codes_match(lib):
    for i, name in enumerate(["ENC_OK", "ENC_ERR_BAD_ARG", "ENC_ERR_UNSUPPORTED", "ENC_ERR_LAUNCH",
                              "ENC_ERR_DEVICE_WAIT", "ENC_ERR_NO_MEMORY"]):
        assert re.search(rf"{name} = {i}\b", HEADER)
    for i, name in enumerate(["F32", "F16", "BF16", "I32", "I8", "I16", "I64", "U8"]):
        assert re.search(rf"ENC_{name} = {i}\b", HEADER) and getattr(N, name) == i


def test_bad_arguments_are_refused_before_any_launch(lib):
    s = lib.enc_softmax(None, None, 4, 4, 4, 4, N.F32, -1, None)
    assert s == N.ERR_BAD_ARG and "NULL" in N.last_error()
    s = lib.enc_softmax(16, 16, 4, 4, 4, 4, 99, -1, None)
    assert s == N.ERR_BAD_ARG and "dtype" in N.last_error()
    s = lib.enc_gelu(16, None, 16, 8, 0, 1.0, 0, 7, N.F32, -1, None)
    assert s == N.ERR_BAD_ARG and "mode" in N.last_error()
    s = lib.enc_histogram(16, 16, 8, 0.0, 1.0, 0, N.I32, -1, None)
    assert s == N.ERR_BAD_ARG
    s = lib.enc_cumsum(16, 16, -1, 4, 4, 4, 0, N.I32, None, -1, None)
    assert s == N.ERR_BAD_ARG
    with pytest.raises(ValueError):
        N.check(s)


def test_empty_problems_are_no_ops(lib):
    assert lib.enc_softmax(16, 16, 0, 128, 128, 128, N.F32, -1, None) == N.OK
    assert lib.enc_gelu(16, None, 16, 0, 0, 1.0, 0, 0, N.F32, -1, None) == N.OK
    assert lib.enc_histogram(None, 16, 0, 0.0, 1.0, 8, N.I32, -1, None) == N.OK
    assert lib.enc_cumsum(None, None, 0, 0, 0, 0, 0, N.I32, None, -1, None) == N.OK


def test_failure_hook_forces_one_failure(lib):
    lib.enc_test_fail_next(N.ERR_LAUNCH)
    assert lib.enc_softmax(16, 16, 0, 0, 0, 0, N.F32, -1, None) == N.ERR_LAUNCH
    assert "injected" in N.last_error()
    with pytest.raises(N.CudaError):
        N.check(N.ERR_LAUNCH)
    assert lib.enc_softmax(16, 16, 0, 0, 0, 0, N.F32, -1, None) == N.OK  # one shot


def test_variant_tables(lib):
    for k in (N.K_SOFTMAX, N.K_LAYERNORM, N.K_RMSNORM, N.K_GELU, N.K_HISTOGRAM, N.K_CUMSUM):
        n = N.num_variants(k)
        assert n >= 1
        assert all(N.variant_info(k, v) for v in range(n))
    with pytest.raises(ValueError):
        N.variant_info(N.K_SOFTMAX, 10_000)
    assert lib.enc_cumsum_out_dtype(N.I8) == N.I32 and lib.enc_cumsum_out_dtype(N.BF16) == N.BF16
