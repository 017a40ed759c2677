"""Regenerates `kernel_bodies.py`: fingerprints of the reference's own kernel bodies.

    python -m enceladus_b200.runtime.make_kernel_bodies /path/to/reference-checkout

The launch path serves a `@jit` kernel by name with a hand-written CUDA kernel and never runs the Python
body.  A body that merely documents the kernel (a docstring, `pass`, `...`) is always accepted; a body with
code is accepted only if it IS one of the reference's kernels of that name, which is what this table
records: for every `@enceladus.jit` function under examples/, benchmarks/ and tests/ of the reference
whose name is in the registry, the SHA-256 of its normalised body (see `jit.body_fingerprint`: the AST of
the statements without the docstring, so that comments and formatting do not matter).  Only fingerprints
are stored, no source text.
"""

from __future__ import annotations

import ast
import sys
from pathlib import Path


def main(ref: str) -> None:
    from enceladus_b200.runtime import registry
    from enceladus_b200.runtime.jit import fingerprint_of_def

    known = set(registry.kernels())
    found: dict[str, set[str]] = {}
    where: dict[str, list[str]] = {}
    root = Path(ref)
    for sub in ("examples", "benchmarks", "tests"):
        for path in sorted((root / sub).rglob("*.py")):
            try:
                tree = ast.parse(path.read_text())
            except SyntaxError:
                continue
            for node in ast.walk(tree):
                if isinstance(node, ast.FunctionDef) and node.name in known and node.decorator_list:
                    params = tuple(a.arg for a in node.args.args)
                    if params != registry._REGISTRY[node.name].params:
                        continue  # same name, another signature: the registry refuses it by its parameter list
                    fp = fingerprint_of_def(node)
                    if fp is None:
                        continue
                    if fp not in found.setdefault(node.name, set()):
                        found[node.name].add(fp)
                        where.setdefault(node.name, []).append(f"{path.relative_to(root)}:{node.lineno}")
    out = Path(__file__).with_name("kernel_bodies.py")
    lines = ['"""Fingerprints of the reference\'s kernel bodies, by kernel name (written by make_kernel_bodies.py)."""',
             "", "KNOWN_BODIES: dict[str, frozenset[str]] = {"]
    for name in sorted(found):
        lines.append(f"    # {', '.join(where[name])}")
        lines.append(f"    {name!r}: frozenset({{")
        for fp in sorted(found[name]):
            lines.append(f"        {fp!r},")
        lines.append("    }),")
    lines.append("}")
    out.write_text("\n".join(lines) + "\n")
    print(f"wrote {out} ({sum(len(v) for v in found.values())} bodies of {len(found)} kernels)")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
