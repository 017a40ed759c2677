"""`Config`, `@autotune` and `@heuristics`.

Same surface and selection rule as the reference autotuner (src/enceladus/runtime/autotuner.py): every
candidate is timed, the fastest few are timed again in interleaved rounds, and among the candidates
within `tolerance` of the fastest the EARLIEST in the list wins; winners are kept per key in memory and
in a JSON file under the cache directory (written under a file lock with an atomic replace).

A candidate here selects one of the hand-written tile variants of the CUDA kernel (`Config.variant`)
in addition to the constexpr values the launch grid depends on (`BM`, `BLOCK_M`, ...).  The Apple
launch options (`num_warps`, `dot_warps`, `dot_backend`) are carried for compatibility and ignored by
the kernels.  Timing uses CUDA events on device-resident copies of the arguments.
"""

from __future__ import annotations

import contextlib
import fcntl
import hashlib
import json
import logging
import os
import statistics
import tempfile
import threading
import time
import warnings
from collections.abc import Callable, Iterable, Sequence
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

import numpy as np

from enceladus_b200.runtime import interop
from enceladus_b200.runtime.jit import JITFunction

log = logging.getLogger("enceladus.autotune")

FINALISTS = 3          # candidates re-timed in phase 2
FINALIST_BAND = 0.15   # ... if within 15% of the fastest
FINAL_ROUNDS = 4
TUNING_VERSION = "b200-1"


def cache_dir() -> Path:
    """`$ENCELADUS_CACHE_DIR` or `~/.cache/enceladus` (src/enceladus/runtime/cache.py)."""
    d = os.environ.get("ENCELADUS_CACHE_DIR")
    return Path(d) if d else Path.home() / ".cache" / "enceladus"


def write_atomic(path: Path, text: str) -> None:
    fd, tmp = tempfile.mkstemp(dir=path.parent, prefix=path.name, suffix=".tmp")
    try:
        with os.fdopen(fd, "w") as f:
            f.write(text)
        os.replace(tmp, path)
    except BaseException:
        with contextlib.suppress(OSError):
            os.unlink(tmp)
        raise


@dataclass
class Config:
    """One candidate: constexpr values, launch options, and the CUDA tile variant.

    Args:
        kwargs: Constexpr values, for example `{"BM": 128, "BN": 256, "BK": 64}`.
        num_warps, dot_warps, dot_backend: Apple launch options, kept for compatibility.
        pre_hook: Called with the bound arguments before each launch of this config.
        variant: Index of the hand-written tile variant (None = the library's own choice).
    """

    kwargs: dict[str, Any]
    num_warps: int = 4
    dot_warps: tuple[int, int] | None = None
    dot_backend: str = "auto"
    pre_hook: Callable[[dict[str, Any]], None] | None = field(default=None, repr=False)
    variant: int | None = None

    def __post_init__(self) -> None:
        if self.dot_backend not in ("auto", "simdgroup", "mpp"):
            raise ValueError(f"dot_backend must be 'auto', 'simdgroup', or 'mpp', not {self.dot_backend!r}")
        if self.dot_warps is not None:
            self.dot_warps = tuple(self.dot_warps)

    def launch_options(self) -> dict[str, Any]:
        opts: dict[str, Any] = {"num_warps": self.num_warps}
        if self.dot_warps is not None:
            opts["dot_warps"] = self.dot_warps
        if self.dot_backend != "auto":
            opts["dot_backend"] = self.dot_backend
        if self.variant is not None:
            opts["variant"] = self.variant
        return opts

    def __str__(self) -> str:
        parts = [repr(self.kwargs), f"num_warps={self.num_warps}"]
        if self.dot_warps is not None:
            parts.append(f"dot_warps={self.dot_warps}")
        if self.dot_backend != "auto":
            parts.append(f"dot_backend={self.dot_backend!r}")
        if self.variant is not None:
            parts.append(f"variant={self.variant}")
        return f"enceladus.Config({', '.join(parts)})"

    def to_json(self) -> dict[str, Any]:
        return {"kwargs": self.kwargs, "num_warps": self.num_warps,
                "dot_warps": list(self.dot_warps) if self.dot_warps else None,
                "dot_backend": self.dot_backend, "variant": self.variant}

    @classmethod
    def from_json(cls, d: dict[str, Any]) -> Config:
        dw = d.get("dot_warps")
        return cls(dict(d["kwargs"]), d["num_warps"], tuple(dw) if dw else None,
                   d.get("dot_backend", "auto"), None, d.get("variant"))

    def _identity(self) -> str:
        return json.dumps(self.to_json(), sort_keys=True)


def _innermost(fn: Any) -> JITFunction:
    while not isinstance(fn, JITFunction):
        inner = getattr(fn, "fn", None)
        if inner is None:
            raise TypeError(f"expected a @enceladus.jit kernel, but got {type(fn).__name__}")
        fn = inner
    return fn


def _named_args(jit: JITFunction, args: tuple, kwargs: dict[str, Any]) -> dict[str, Any]:
    named = dict(zip(jit.arg_names, args))
    named.update(kwargs)
    return named


class Heuristics:
    """Computes constexpr values from the other arguments. Created by `@heuristics`."""

    def __init__(self, fn: Any, values: dict[str, Callable[[dict[str, Any]], Any]]) -> None:
        self.fn, self.values = fn, values
        self.jit = _innermost(fn)
        self.arg_names = self.jit.arg_names

    def resolve(self, args: tuple, kwargs: dict[str, Any]) -> dict[str, Any]:
        named = _named_args(self.jit, args, kwargs)
        return {**kwargs, **{k: f(named) for k, f in self.values.items()}}

    def __getitem__(self, grid: Any) -> Callable[..., None]:
        return lambda *args, **kwargs: self.run(*args, grid=grid, **kwargs)

    def run(self, *args: Any, grid: Any, **kwargs: Any) -> None:
        self.fn.run(*args, grid=grid, **self.resolve(args, kwargs))


def heuristics(values: dict[str, Callable[[dict[str, Any]], Any]]):
    """Decorates a kernel so that constexpr values come from functions of the arguments."""
    return lambda fn: Heuristics(fn, values)


def _key_value(v: Any) -> str:
    return repr(v.item() if isinstance(v, np.generic) else v)


def _key_dtype(v: Any) -> str | None:
    return str(interop.element_dtype(v)) if interop.is_array(v) else None


def _device_view(v: Any) -> Any:
    """A device-resident stand-in for an argument, so that timing excludes host copies."""
    if isinstance(v, np.ndarray):
        return interop._np_as_torch_view(np.ascontiguousarray(v)).to("cuda")
    return v


class Autotuner:
    """Picks the fastest `Config` per key. Created by `@autotune`."""

    def __init__(self, fn: Any, configs: Sequence[Config], key: Sequence[str],
                 prune_configs_by: dict[str, Callable] | None = None,
                 reset_to_zero: Iterable[str] | None = None, restore_value: Iterable[str] | None = None,
                 warmup_ms: float = 50, rep: int = 20, tolerance: float = 0.01) -> None:
        if not configs:
            raise ValueError("@enceladus.autotune needs at least one Config")
        if not 0 <= tolerance < 1:
            raise ValueError(f"tolerance must be in [0, 1), but got {tolerance}")
        self.tolerance = tolerance
        self.fn = fn
        self.jit = _innermost(fn)
        self.configs = list(configs)
        self.key = list(key)
        self.prune = prune_configs_by or {}
        self.reset_to_zero = list(reset_to_zero or [])
        self.restore_value = list(restore_value or [])
        self.warmup_ms, self.rep = warmup_ms, rep
        self.arg_names = self.jit.arg_names
        for k in (*self.key, *self.reset_to_zero, *self.restore_value):
            if k not in self.arg_names:
                raise ValueError(f"@enceladus.autotune names unknown argument {k!r}")
        self.best: dict[str, Config] = {}
        self._saved: dict[str, Config] = {}
        self.timings: dict[str, dict[str, float]] = {}
        self._loaded = False
        self._lock = threading.Lock()

    # ---- persistence ----
    def _arch(self) -> str:
        try:
            from enceladus_b200 import _native

            info = _native.device_info()
            return f"sm_{info.cc_major}{info.cc_minor}a-{info.name.decode().replace(' ', '_')}"
        except Exception:  # noqa: BLE001 - no device: results are not device specific
            return "unknown"

    def _path(self) -> Path:
        ident = hashlib.sha256("|".join([self.jit.__name__, ",".join(self.arg_names), TUNING_VERSION])
                               .encode()).hexdigest()[:32]
        return cache_dir() / "autotune" / ident / f"{self._arch()}.json"

    def _load(self) -> None:
        self._loaded = True
        if os.environ.get("ENCELADUS_ALWAYS_COMPILE", "0") not in ("", "0"):
            return
        try:
            data = json.loads(self._path().read_text())
        except (OSError, ValueError):
            return
        if not isinstance(data, dict):
            return
        for k, v in data.items():
            try:
                self._saved.setdefault(k, Config.from_json(v))
            except (KeyError, TypeError, ValueError):
                log.debug("ignoring malformed saved result %r for key %s", v, k)

    def _from_saved(self, key: str, named: dict[str, Any]) -> Config | None:
        saved = self._saved.pop(key, None)
        if saved is None:
            return None
        ident = saved._identity()
        return next((c for c in self._candidates(named) if c._identity() == ident), None)

    def _save(self) -> None:
        p = self._path()
        try:
            p.parent.mkdir(parents=True, exist_ok=True)
            with open(p.with_suffix(".lock"), "a") as lock:
                fcntl.flock(lock, fcntl.LOCK_EX)
                data: dict[str, Any] = {}
                with contextlib.suppress(OSError, ValueError):
                    loaded = json.loads(p.read_text())
                    if isinstance(loaded, dict):
                        data = loaded
                data.update({k: c.to_json() for k, c in self.best.items()})
                write_atomic(p, json.dumps(data, indent=1, sort_keys=True))
        except OSError as e:
            log.debug("couldn't save autotuning results: %s", e)

    # ---- tuning ----
    def _key(self, named: dict[str, Any]) -> str:
        parts = [_key_value(named[k]) for k in self.key]
        dtypes = [d for n in self.arg_names if (d := _key_dtype(named.get(n))) is not None]
        return "|".join(parts) + "|" + ",".join(dtypes)

    def __getitem__(self, grid: Any) -> Callable[..., None]:
        return lambda *args, **kwargs: self.run(*args, grid=grid, **kwargs)

    def config_for(self, *args: Any, **kwargs: Any) -> Config | None:
        """The tuned config for these launch arguments, or None if not tuned yet."""
        return self.best.get(self._key(_named_args(self.jit, args, kwargs)))

    def run(self, *args: Any, grid: Any, **kwargs: Any) -> None:
        if not self._loaded:
            self._load()
        named = _named_args(self.jit, args, kwargs)
        key = self._key(named)
        cfg = self.best.get(key)
        if cfg is None:
            with self._lock:
                cfg = self.best.get(key) or self._from_saved(key, named)
                if cfg is None:
                    cfg = self._tune(key, args, kwargs, grid, named)
                self.best[key] = cfg
        if cfg.pre_hook is not None:
            cfg.pre_hook(named)
        self.fn.run(*args, grid=grid, **kwargs, **cfg.kwargs, **cfg.launch_options())

    def _candidates(self, named: dict[str, Any]) -> list[Config]:
        configs = self.configs
        early = self.prune.get("early_config_prune")
        if early is not None:
            configs = list(early(configs, named))
        model, top_k = self.prune.get("perf_model"), self.prune.get("top_k")
        if model is not None and top_k:
            scored = sorted(configs, key=lambda c: model(**{**named, **c.kwargs}, num_warps=c.num_warps))
            n = int(top_k * len(configs)) if isinstance(top_k, float) else int(top_k)
            configs = scored[: max(1, n)]
        return configs

    def _tune(self, key: str, args: tuple, kwargs: dict, grid: Any, named: dict) -> Config:
        from enceladus_b200.testing import do_bench

        start = time.perf_counter()
        configs = self._candidates(named)
        bench_args = tuple(_device_view(a) for a in args)
        bench_kwargs = {k: _device_view(v) for k, v in kwargs.items()}
        named_bench = _named_args(self.jit, bench_args, bench_kwargs)
        saved = {n: named_bench[n].clone() for n in self.restore_value if interop.is_torch(named_bench.get(n))}
        errors: dict[int, Exception] = {}

        def launch(cfg: Config) -> None:
            for n, v in saved.items():
                named_bench[n].copy_(v)
            for n in self.reset_to_zero:
                if interop.is_torch(named_bench.get(n)):
                    named_bench[n].zero_()
            if cfg.pre_hook is not None:
                cfg.pre_hook(named_bench)
            self.fn.run(*bench_args, grid=grid, **bench_kwargs, **cfg.kwargs, **cfg.launch_options())

        def bench(i: int, warmup_ms: float, rep: int, mode: str) -> Any:
            try:
                return do_bench(lambda: launch(configs[i]), warmup_ms, rep, mode)
            except Exception as e:  # noqa: BLE001 - a config that fails to launch is skipped
                errors[i] = e
                warnings.warn(f"{self.jit.__name__}: skipping {configs[i]}: {e}", stacklevel=5)
                return None

        timings: dict[int, float] = {}
        for i in range(len(configs)):  # phase 1: every candidate
            if (t := bench(i, self.warmup_ms, self.rep, "median")) is not None:
                timings[i] = t
        order = sorted(timings, key=timings.get)
        finalists = [i for i in order[:FINALISTS] if timings[i] <= timings[order[0]] * (1 + FINALIST_BAND)]
        if len(finalists) > 1:  # phase 2: interleaved rounds, first sample after a switch dropped
            per_round = max(3, self.rep // 4)
            samples: dict[int, list[float]] = {i: [] for i in finalists}
            for _ in range(FINAL_ROUNDS):
                for i in finalists:
                    if i not in errors and (s := bench(i, 0, per_round + 1, "all")) is not None:
                        samples[i] += s[1:]
            for i in list(finalists):
                if i in errors or not samples[i]:
                    timings.pop(i, None)
                else:
                    timings[i] = statistics.median(samples[i])
            finalists = [i for i in finalists if i in timings]
        for n, v in saved.items():
            named_bench[n].copy_(v)
        for n in self.reset_to_zero:
            if interop.is_torch(named_bench.get(n)):
                named_bench[n].zero_()
        if not timings:
            first = next(iter(errors.values()))
            raise RuntimeError(f"every autotuning config of {self.jit.__name__} failed to run; the first "
                               f"error was: {first}") from first
        pool = finalists if len(finalists) > 1 else list(timings)
        fastest = min(timings[i] for i in pool)
        best_i = min(i for i in pool if timings[i] <= fastest * (1 + self.tolerance))
        best = configs[best_i]
        self.best[key] = best
        self.timings[key] = {str(configs[i]): t for i, t in timings.items()}
        self._save()
        elapsed = time.perf_counter() - start
        if os.environ.get("ENCELADUS_PRINT_AUTOTUNING", "0") not in ("", "0"):
            print(f"enceladus: autotuning {self.jit.__name__} [{key}] chose {best} "
                  f"({timings[best_i]:.3f} ms, tuned in {elapsed:.1f} s)")
        return best


def autotune(configs: Sequence[Config], key: Sequence[str], prune_configs_by: dict[str, Callable] | None = None,
             reset_to_zero: Iterable[str] | None = None, restore_value: Iterable[str] | None = None,
             warmup_ms: float = 50, rep: int = 20, tolerance: float = 0.01):
    """Decorates a kernel so that each launch uses the fastest of `configs` (autotuner.py:549-585)."""
    return lambda fn: Autotuner(fn, configs, key, prune_configs_by, reset_to_zero, restore_value,
                                warmup_ms, rep, tolerance)
