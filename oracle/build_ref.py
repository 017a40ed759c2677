"""Installs the reference's own CPU path into `oracle/_ref/` so that it can be timed and used as a checker
on a machine that has no reference checkout (the GPU box).

    python oracle/build_ref.py [--reference /path/to/enceladus-checkout] [--out oracle/_ref]

TEST AND MEASUREMENT INFRASTRUCTURE ONLY: nothing under `enceladus_b200/` imports what this installs.  Users
are `tests/`, `bench.py`'s CPU-baseline legs / `--impl reference`, and `__graft_entry__.build()`, which runs
this recipe whenever a checkout is present.

The reference is a pure-Python project; its CPU implementation of the kernel path is its NumPy interpreter
(`ENCELADUS_INTERPRET=1`: src/enceladus/runtime/jit.py:398-418 -> src/enceladus/interpreter/interp.py:801-825)
and each example's float64 `reference()` (examples/02_softmax.py:41, 03_layernorm.py:60, 07_matmul_fused.py:54,
08_flash_attention.py:130, 09_histogram.py:37, 10_cumsum.py:45).  "Building" it is therefore an install, the
same thing `pip install --target` does: the package's files (minus the `_C` sources) and the example modules are copied,
unmodified, from where they lie in the checkout into the output directory, which `.gitignore` lists (no
reference source enters the history; the directory travels to the GPU box like a built `.so`).  The one file
written here rather than copied is `enceladus/_C.py`: a placeholder for the Metal extension the package
imports at start-up (`from enceladus._C import MetalError`, src/enceladus/__init__.py:12), which cannot be
built on Linux and which the interpreter path never calls.
"""

from __future__ import annotations

import argparse
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEFAULT_REFERENCE = Path("/root/reference")

STUB = '''"""Placeholder for the reference's Metal extension (src/enceladus/_C/*.mm), written by oracle/build_ref.py.
The interpreter path imports these names and never instantiates them."""


class MetalError(RuntimeError):
    pass


class _Handle:
    def __init__(self, *args, **kwargs):
        raise MetalError("the Metal runtime is not available here; only ENCELADUS_INTERPRET=1 works")


class Buffer(_Handle): ...
class Pipeline(_Handle): ...
class Queue(_Handle): ...
class Stream(_Handle): ...
class LaunchPlan(_Handle): ...
class Device(_Handle): ...
class Library(_Handle): ...
'''


def build(reference: Path | str = DEFAULT_REFERENCE, out: Path | str = HERE / "_ref", quiet: bool = False) -> bool:
    """Returns True when `out` holds an importable install afterwards; False when there is no checkout."""
    reference, out = Path(reference), Path(out)
    pkg, examples = reference / "src" / "enceladus", reference / "examples"
    if not (pkg / "__init__.py").exists():
        return (out / "enceladus" / "__init__.py").exists()
    if out.exists():
        shutil.rmtree(out)
    skip = shutil.ignore_patterns("__pycache__", "*.pyc", "_C")  # package data (the .metal prelude read at import) stays
    shutil.copytree(pkg, out / "enceladus", ignore=skip)
    (out / "enceladus" / "_C.py").write_text(STUB)
    (out / "examples").mkdir()
    for f in sorted(examples.glob("*.py")):
        shutil.copy2(f, out / "examples" / f.name)
    n = sum(1 for _ in out.rglob("*.py"))
    (out / "INSTALLED_FROM").write_text(f"{reference}\n{n} python files\n")
    if not quiet:
        print(f"installed the reference's CPU path into {out} ({n} files)")
    return True


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=str(DEFAULT_REFERENCE))
    ap.add_argument("--out", default=str(HERE / "_ref"))
    a = ap.parse_args()
    sys.exit(0 if build(a.reference, a.out) else 1)
