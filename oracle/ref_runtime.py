"""Loads the reference's own CPU path from `oracle/_ref/` (installed by `oracle/build_ref.py`).

TEST AND MEASUREMENT INFRASTRUCTURE ONLY: imported by `tests/` and by `bench.py`'s CPU-baseline legs, never
by the product.  `load()` returns None when nothing is installed (callers then fall back to the NumPy
restatement in `enceladus_oracle.py` and say so).

    ref = load()
    y = ref.example("02_softmax").softmax(x)         # runs softmax_kernel under the reference interpreter
    y64 = ref.example("02_softmax").reference(x)     # the example's own float64 NumPy path

The interpreter is selected exactly as a user of the reference selects it: ENCELADUS_INTERPRET=1
(src/enceladus/runtime/jit.py:398-418), with ENCELADUS_VERIFY=0 so that no Metal compile check runs.  The
two variables are set only for the duration of a call into the reference (`interpreting()`), because the
CUDA package in the same process refuses to launch while ENCELADUS_INTERPRET asks for an interpreter.
"""

from __future__ import annotations

import contextlib
import functools
import importlib
import importlib.util
import os
import sys
import types
from pathlib import Path

ROOT = Path(__file__).resolve().parent / "_ref"


@contextlib.contextmanager
def interpreting():
    """ENCELADUS_INTERPRET=1 and ENCELADUS_VERIFY=0 for the enclosed calls; the previous values come back after."""
    old = {k: os.environ.get(k) for k in ("ENCELADUS_INTERPRET", "ENCELADUS_VERIFY")}
    os.environ["ENCELADUS_INTERPRET"], os.environ["ENCELADUS_VERIFY"] = "1", "0"
    try:
        yield
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


class _Interpreted:
    """An example module whose functions run under `interpreting()`."""

    def __init__(self, module: types.ModuleType) -> None:
        self._module = module

    def __getattr__(self, name: str):
        attr = getattr(self._module, name)
        if not isinstance(attr, types.FunctionType):
            return attr

        @functools.wraps(attr)
        def call(*args, **kwargs):
            with interpreting():
                return attr(*args, **kwargs)

        return call


class Reference:
    def __init__(self, root: Path) -> None:
        self.root = root
        self._examples: dict[str, object] = {}
        if str(root) not in sys.path:
            sys.path.insert(0, str(root))
        with interpreting():
            self.package = importlib.import_module("enceladus")

    def example(self, name: str):
        """Module object of examples/<name>.py (e.g. "03_layernorm"); the file names start with a digit, so they
        are loaded by path."""
        mod = self._examples.get(name)
        if mod is None:
            path = self.root / "examples" / f"{name}.py"
            spec = importlib.util.spec_from_file_location(f"enceladus_ref_example_{name}", path)
            raw = importlib.util.module_from_spec(spec)
            with interpreting():
                spec.loader.exec_module(raw)
            mod = self._examples[name] = _Interpreted(raw)
        return mod


_cached: Reference | None = None


def available() -> bool:
    return (ROOT / "enceladus" / "__init__.py").exists() and (ROOT / "enceladus" / "_C.py").exists()


def load() -> Reference | None:
    global _cached
    if _cached is None and available():
        _cached = Reference(ROOT)
    return _cached
