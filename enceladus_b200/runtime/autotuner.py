"""`Config`, `@autotune` and `@heuristics`: choosing among the hand-written tile variants of a kernel.

The public surface is the reference's (src/enceladus/runtime/autotuner.py:53-109, 549-585): `Config(kwargs,
num_warps, dot_warps, dot_backend, pre_hook)`, `autotune(configs, key, prune_configs_by, reset_to_zero,
restore_value, warmup_ms, rep, tolerance)`, `heuristics(values)`, `tuned[grid](...)`, `config_for(...)`, one
result per key (the `key` argument values plus the element types of the array arguments), results kept in a
JSON file under `$ENCELADUS_CACHE_DIR`, and the selection rule: among the candidates within `tolerance` of the
fastest, the EARLIEST in the list wins, so that the order of `configs` expresses a preference.

What is tuned is different, and the machinery follows from that.  A candidate here does not compile anything:
it names one precompiled variant of a CUDA kernel (`Config.variant`), so trying a candidate costs one launch.
The tuner therefore races all candidates against each other in interleaved passes (every pass times each
survivor once, so clock and thermal drift hit all of them alike), times each launch by itself with a pair of
CUDA events (what `restore_value` / `reset_to_zero` / `pre_hook` do between launches is not in the figure) and
drops a candidate as soon as its best pass is out of reach of the leader.  A saved result is only valid for
the library build whose variant numbering it refers to: the file records a digest of the variant
descriptions (`enc_variant_info`) and is ignored when that changes.
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

PASSES = 5            # interleaved passes over the surviving candidates
OUT_OF_REACH = 1.15   # a candidate whose best pass is this much slower than the leader's median leaves the race
_BACKENDS = ("auto", "simdgroup", "mpp")


def cache_dir() -> Path:
    """`$ENCELADUS_CACHE_DIR` or `~/.cache/enceladus` (src/enceladus/runtime/cache.py)."""
    d = os.environ.get("ENCELADUS_CACHE_DIR")
    return Path(d) if d else Path.home() / ".cache" / "enceladus"


def _env_on(name: str) -> bool:
    return os.environ.get(name, "0") not in ("", "0")


# ---- candidates ----------------------------------------------------------------------------------------
@dataclass
class Config:
    """One candidate: constexpr values, launch options, and the CUDA tile variant.

    Args:
        kwargs: Constexpr values, for example `{"BM": 128, "BN": 256, "BK": 64}`; the launch grid is usually
            computed from them, so they must describe the tile the variant really uses.
        num_warps, dot_warps, dot_backend: the reference's Apple launch options; accepted, validated and passed
            on, without effect on the CUDA kernels.
        pre_hook: Called with the bound arguments before each launch of this config.
        variant: Index of the hand-written tile variant (None = the library's own choice).
    """

    kwargs: dict[str, Any]
    num_warps: int = 4
    dot_warps: tuple[int, int] | None = None
    dot_backend: str = "auto"
    pre_hook: Callable[[dict[str, Any]], None] | None = field(default=None, repr=False, compare=False)
    variant: int | None = None

    def __post_init__(self) -> None:
        if self.dot_backend not in _BACKENDS:
            raise ValueError(f"dot_backend must be 'auto', 'simdgroup', or 'mpp', not {self.dot_backend!r}")
        self.dot_warps = None if self.dot_warps is None else tuple(self.dot_warps)

    def launch_options(self) -> dict[str, Any]:
        """Keyword arguments of `kernel.run` that this candidate adds beside its constexpr values."""
        opts = {"num_warps": self.num_warps, "dot_warps": self.dot_warps, "variant": self.variant,
                "dot_backend": None if self.dot_backend == "auto" else self.dot_backend}
        return {k: v for k, v in opts.items() if v is not None}

    def __str__(self) -> str:
        extra = "".join(f", {k}={v!r}" for k, v in self.launch_options().items())
        return f"enceladus.Config({self.kwargs!r}{extra})"

    def to_json(self) -> dict[str, Any]:
        return {"kwargs": dict(self.kwargs), "variant": self.variant, "num_warps": self.num_warps,
                "dot_warps": None if self.dot_warps is None else list(self.dot_warps), "dot_backend": self.dot_backend}

    @classmethod
    def from_json(cls, record: dict[str, Any]) -> Config:
        return cls(dict(record["kwargs"]), num_warps=record.get("num_warps", 4), dot_warps=record.get("dot_warps"),
                   dot_backend=record.get("dot_backend", "auto"), variant=record.get("variant"))

    def tag(self) -> str:
        """A canonical string: two configs with the same tag launch the same thing."""
        return json.dumps(self.to_json(), sort_keys=True, default=repr)


def _jit_of(fn: Any) -> JITFunction:
    """The `@jit` kernel under a stack of decorators (`Heuristics`, `Autotuner`)."""
    seen = fn
    while not isinstance(seen, JITFunction):
        seen = getattr(seen, "fn", None)
        if seen is None:
            raise TypeError(f"expected a @enceladus.jit kernel, but got {type(fn).__name__}")
    return seen


def _by_name(jit: JITFunction, args: tuple, kwargs: dict[str, Any]) -> dict[str, Any]:
    return {**dict(zip(jit.arg_names, args)), **kwargs}


class Heuristics:
    """Computes constexpr values from the other arguments. Created by `@heuristics`."""

    def __init__(self, fn: Any, values: dict[str, Callable[[dict[str, Any]], Any]]) -> None:
        self.fn, self.values = fn, dict(values)
        self.jit = _jit_of(fn)
        self.arg_names = self.jit.arg_names

    def __getitem__(self, grid: Any) -> Callable[..., None]:
        return lambda *args, **kwargs: self.run(*args, grid=grid, **kwargs)

    def run(self, *args: Any, grid: Any, **kwargs: Any) -> None:
        seen = _by_name(self.jit, args, kwargs)
        computed = {name: rule(seen) for name, rule in self.values.items()}
        self.fn.run(*args, grid=grid, **{**kwargs, **computed})


def heuristics(values: dict[str, Callable[[dict[str, Any]], Any]]):
    """Decorates a kernel so that constexpr values come from functions of the arguments."""
    return lambda fn: Heuristics(fn, values)


# ---- what a result depends on -----------------------------------------------------------------------------
def device_tag() -> str:
    """Names the GPU model a result was measured on (one result file per model)."""
    try:
        from enceladus_b200 import _native

        info = _native.device_info()
        return f"sm_{info.cc_major}{info.cc_minor}-{info.name.decode().replace(' ', '_')}-{info.sm_count}sm"
    except Exception:  # noqa: BLE001 - no device or no library: nothing device specific can be said
        return "no-device"


def library_digest(jit: JITFunction) -> str:
    """Digest of the variant descriptions of the kernel this `@jit` function launches.  `Config.variant` is an index
    into that list, so a saved winner means something only while the list is the same."""
    try:
        from enceladus_b200 import _native

        kernel_id = jit.adapter().kernel_id
        lines = [_native.variant_info(kernel_id, v) for v in range(_native.num_variants(kernel_id))]
    except Exception:  # noqa: BLE001 - unknown kernel or no library (host-only use): nothing to index
        lines = []
    return hashlib.sha256("\n".join(lines).encode()).hexdigest()[:16]


def time_launches(launch: Callable[[], None], count: int) -> list[float]:
    """Milliseconds of each of `count` launches, each bracketed by its own pair of CUDA events on the current
    stream.  Without a CUDA device (host-only tests with stand-in kernels) wall-clock time is used."""
    torch = interop._torch()
    if not torch.cuda.is_available():
        out = []
        for _ in range(count):
            t0 = time.perf_counter()
            launch()
            out.append((time.perf_counter() - t0) * 1e3)
        return out
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(count)]
    for begin, end in pairs:
        begin.record()
        launch()
        end.record()
    torch.cuda.synchronize()
    return [b.elapsed_time(e) for b, e in pairs]


def on_device(value: Any) -> Any:
    """NumPy arguments are replaced by device copies while tuning, so that no candidate is charged for staging."""
    if isinstance(value, np.ndarray):
        return interop._np_as_torch_view(np.ascontiguousarray(value)).to("cuda")
    return value


class _Store:
    """The JSON file that keeps winners across processes: {"library": digest, "results": {key: {config, ms}}}."""

    def __init__(self, jit: JITFunction) -> None:
        self.jit = jit

    def path(self) -> Path:
        sig = hashlib.sha256(",".join(self.jit.arg_names).encode()).hexdigest()[:12]
        return cache_dir() / "autotune" / f"{self.jit.__name__}-{sig}" / f"{device_tag()}.json"

    def read(self) -> dict[str, Config]:
        try:
            doc = json.loads(self.path().read_text())
            if doc.get("library") != library_digest(self.jit):
                return {}
            return {key: Config.from_json(rec["config"]) for key, rec in doc.get("results", {}).items()}
        except (OSError, ValueError, KeyError, TypeError, AttributeError):
            return {}

    def merge(self, winners: dict[str, tuple[Config, float]]) -> None:
        """Adds `winners` to the file under an exclusive lock; the file is replaced atomically."""
        path = self.path()
        try:
            path.parent.mkdir(parents=True, exist_ok=True)
            with open(path.with_suffix(".lock"), "a") as guard:
                fcntl.flock(guard, fcntl.LOCK_EX)
                digest = library_digest(self.jit)
                doc = {"library": digest, "results": {}}
                with contextlib.suppress(OSError, ValueError):
                    old = json.loads(path.read_text())
                    if isinstance(old, dict) and old.get("library") == digest and isinstance(old.get("results"), dict):
                        doc["results"] = old["results"]
                for key, (cfg, ms) in winners.items():
                    doc["results"][key] = {"config": cfg.to_json(), "ms": ms}
                fd, tmp = tempfile.mkstemp(dir=path.parent, prefix=path.name, suffix=".tmp")
                with os.fdopen(fd, "w") as f:
                    json.dump(doc, f, indent=1, sort_keys=True)
                os.replace(tmp, path)
        except OSError as e:
            log.debug("autotuning results not saved: %s", e)


# ---- the tuner -------------------------------------------------------------------------------------------
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
        self.fn, self.jit = fn, _jit_of(fn)
        self.arg_names = self.jit.arg_names
        self.configs, self.key = list(configs), list(key)
        self.prune = dict(prune_configs_by or {})
        self.reset_to_zero, self.restore_value = list(reset_to_zero or ()), list(restore_value or ())
        unknown = [n for n in (*self.key, *self.reset_to_zero, *self.restore_value) if n not in self.arg_names]
        if unknown:
            raise ValueError(f"@enceladus.autotune names unknown argument {unknown[0]!r}")
        self.warmup_ms, self.rep, self.tolerance = warmup_ms, rep, tolerance
        self.best: dict[str, Config] = {}               # key -> winner, this process
        self.timings: dict[str, dict[str, float]] = {}  # key -> {str(config): median ms} of the last race
        self._store = _Store(self.jit)
        self._on_disk: dict[str, Config] | None = None
        self._lock = threading.Lock()

    def __getitem__(self, grid: Any) -> Callable[..., None]:
        return lambda *args, **kwargs: self.run(*args, grid=grid, **kwargs)

    # -- keys and candidates --
    def key_of(self, seen: dict[str, Any]) -> str:
        values = []
        for name in self.key:
            v = seen[name]
            values.append(repr(v.item() if isinstance(v, np.generic) else v))
        dtypes = [str(interop.element_dtype(seen[n])) for n in self.arg_names if n in seen and interop.is_array(seen[n])]
        return "|".join(values) + "|" + ",".join(dtypes)

    def candidates(self, seen: dict[str, Any]) -> list[Config]:
        """`configs` after the user's pruning: `early_config_prune(configs, named_args)`, then the `top_k` best
        by `perf_model(**named_args, **config.kwargs, num_warps=...)` (an int, or a fraction of the list)."""
        pool = list(self.configs)
        if (early := self.prune.get("early_config_prune")) is not None:
            pool = list(early(pool, seen))
        model, top_k = self.prune.get("perf_model"), self.prune.get("top_k")
        if model is not None and top_k:
            keep = max(1, int(top_k * len(pool)) if isinstance(top_k, float) else int(top_k))
            pool = sorted(pool, key=lambda c: model(**{**seen, **c.kwargs}, num_warps=c.num_warps))[:keep]
        return pool

    def config_for(self, *args: Any, **kwargs: Any) -> Config | None:
        """The tuned config for these launch arguments, or None if not tuned yet."""
        return self.best.get(self.key_of(_by_name(self.jit, args, kwargs)))

    # -- launching --
    def run(self, *args: Any, grid: Any, **kwargs: Any) -> None:
        seen = _by_name(self.jit, args, kwargs)
        key = self.key_of(seen)
        cfg = self.best.get(key)
        if cfg is None:
            with self._lock:
                cfg = self.best.get(key) or self._recall(key, seen) or self._race(key, args, kwargs, grid, seen)
                self.best[key] = cfg
        if cfg.pre_hook is not None:
            cfg.pre_hook(seen)
        self.fn.run(*args, grid=grid, **kwargs, **cfg.kwargs, **cfg.launch_options())

    def _recall(self, key: str, seen: dict[str, Any]) -> Config | None:
        """A winner saved by an earlier process, matched back to one of the current candidates (so that hooks, which
        cannot be saved, come from the live object)."""
        if self._on_disk is None:
            self._on_disk = {} if _env_on("ENCELADUS_ALWAYS_COMPILE") else self._store.read()
        saved = self._on_disk.get(key)
        if saved is None:
            return None
        return next((c for c in self.candidates(seen) if c.tag() == saved.tag()), None)

    def _race(self, key: str, args: tuple, kwargs: dict, grid: Any, seen: dict) -> Config:
        started = time.perf_counter()
        field_ = self.candidates(seen)
        dev_args = tuple(on_device(a) for a in args)
        dev_kwargs = {k: on_device(v) for k, v in kwargs.items()}
        dev_seen = _by_name(self.jit, dev_args, dev_kwargs)
        keep = {n: dev_seen[n].clone() for n in self.restore_value if interop.is_torch(dev_seen.get(n))}
        zero = [dev_seen[n] for n in self.reset_to_zero if interop.is_torch(dev_seen.get(n))]

        def prepare(cfg: Config) -> None:  # between launches, outside the timed interval
            for name, value in keep.items():
                dev_seen[name].copy_(value)
            for t in zero:
                t.zero_()
            if cfg.pre_hook is not None:
                cfg.pre_hook(dev_seen)

        def one_pass(cfg: Config, count: int) -> float:
            """Median milliseconds of `count` launches of `cfg`."""
            samples: list[float] = []
            for _ in range(count):
                prepare(cfg)
                samples += time_launches(lambda: self.fn.run(*dev_args, grid=grid, **dev_kwargs, **cfg.kwargs,
                                                             **cfg.launch_options()), 1)
            return statistics.median(samples)

        # every candidate once, untimed: a candidate that cannot launch leaves here; then the clocks get their ramp
        alive: list[int] = []
        failures: list[Exception] = []
        for i, cfg in enumerate(field_):
            try:
                one_pass(cfg, 1)
                alive.append(i)
            except Exception as e:  # noqa: BLE001 - a config that fails to launch is skipped
                failures.append(e)
                warnings.warn(f"{self.jit.__name__}: skipping {cfg}: {e}", stacklevel=4)
        if not alive:
            raise RuntimeError(f"every autotuning config of {self.jit.__name__} failed to run; the first "
                               f"error was: {failures[0]}") from failures[0]
        ramp_until = time.perf_counter() + self.warmup_ms * 1e-3
        while len(alive) > 1 and time.perf_counter() < ramp_until:
            one_pass(field_[alive[0]], 1)

        per_pass = max(3, self.rep // PASSES)
        history: dict[int, list[float]] = {i: [] for i in alive}
        for _ in range(PASSES if len(alive) > 1 else 1):
            for i in list(alive):
                try:
                    history[i].append(one_pass(field_[i], per_pass))
                except Exception as e:  # noqa: BLE001 - fails only under timing (e.g. out of memory with the clones alive)
                    alive.remove(i)
                    warnings.warn(f"{self.jit.__name__}: skipping {field_[i]}: {e}", stacklevel=4)
            if not alive:
                raise RuntimeError(f"every autotuning config of {self.jit.__name__} failed to run")
            lead = min(statistics.median(history[i]) for i in alive)
            alive = [i for i in alive if min(history[i]) <= lead * OUT_OF_REACH]
            if len(alive) == 1:
                break
        prepare(field_[alive[0]])  # leave the caller's buffers as restore_value / reset_to_zero promise

        score = {i: statistics.median(history[i]) for i in history if history[i]}
        fastest = min(score[i] for i in alive)
        winner = min(i for i in alive if score[i] <= fastest * (1 + self.tolerance))  # earliest within tolerance
        best = field_[winner]
        self.best[key] = best
        self.timings[key] = {str(field_[i]): ms for i, ms in score.items()}
        self._store.merge({key: (best, score[winner])})
        if _env_on("ENCELADUS_PRINT_AUTOTUNING"):
            print(f"enceladus: autotuning {self.jit.__name__} [{key}] chose {best} "
                  f"({score[winner]:.3f} ms, {len(field_)} candidates, {time.perf_counter() - started:.1f} s)")
        return best


def autotune(configs: Sequence[Config], key: Sequence[str], prune_configs_by: dict[str, Callable] | None = None,
             reset_to_zero: Iterable[str] | None = None, restore_value: Iterable[str] | None = None,
             warmup_ms: float = 50, rep: int = 20, tolerance: float = 0.01):
    """Decorates a kernel so that each launch uses the fastest of `configs` (autotuner.py:549-585)."""
    return lambda fn: Autotuner(fn, configs, key, prune_configs_by, reset_to_zero, restore_value,
                                warmup_ms, rep, tolerance)
