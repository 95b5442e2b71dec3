"""Autotuner: pick the fastest of several launch configurations, per problem key.

The reference has no tuner — constexpr values are whatever the caller passes
(e.g. ``BLOCK=block`` in tests/test_long_row_sum_kernel.py:64).  This adds the
familiar decorator form:

    @triton.autotune(
        configs=[triton.Config({"BLOCK": 1024}, num_warps=4),
                 triton.Config({"BLOCK": 4096}, num_warps=8)],
        key=["n"])
    @triton.jit
    def kernel(x, out, n, BLOCK: tl.constexpr): ...

A ``Config`` carries constexpr values plus backend knobs (``num_warps``,
``num_stages``, ``online_softmax``, ``elems_per_thread``).  On the first call
for a given key (the values of the ``key`` arguments and the dtypes of the array
arguments) every config is compiled and timed on the device with CUDA events,
on the caller's buffers; the winner is cached in memory and, if
``cache_path`` is set, in a JSON file.  Host (NumPy) arguments are compile-only,
so the first config is used and nothing is timed.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Sequence

from . import arrays
from .compiler import BACKEND_OPTIONS, CompiledKernel, Grid


@dataclass(frozen=True)
class Config:
    kwargs: dict[str, Any] = field(default_factory=dict)
    num_warps: int | None = None
    num_stages: int | None = None
    online_softmax: bool | None = None
    elems_per_thread: int | None = None
    cta_group: int | None = None
    min_ctas_per_sm: int | None = None
    group_m: int | None = None
    tensor_cores: bool | None = None
    a_rows: int | None = None
    loop_passes: bool | None = None
    cta_rows: int | None = None
    bounds_check: bool | None = None
    tile_n: int | None = None
    split_k: int | None = None

    def all_kwargs(self) -> dict[str, Any]:
        merged = dict(self.kwargs)
        for name in BACKEND_OPTIONS:
            value = getattr(self, name, None)
            if value is not None:
                merged[name] = value
        return merged

    def label(self) -> str:
        return ", ".join(f"{k}={v}" for k, v in self.all_kwargs().items())

    def __hash__(self) -> int:
        return hash(tuple(sorted(self.all_kwargs().items())))


def device_timer(run: Callable[[], None], stream_of: Callable[[], int], warmup: int, rep: int) -> float:
    """Milliseconds per launch, CUDA events on the launching stream."""
    from . import runtime

    for _ in range(warmup):
        run()
    start, stop = runtime.Event(), runtime.Event()
    stream = stream_of()
    start.record(stream)
    for _ in range(rep):
        run()
    stop.record(stream)
    stop.synchronize()
    elapsed = start.elapsed_ms(stop) / rep
    start.close()
    stop.close()
    return elapsed


class Autotuner:
    def __init__(self, kernel: CompiledKernel, configs: Sequence[Config], key: Sequence[str],
                 warmup: int = 2, rep: int = 5, cache_path: str | os.PathLike | None = None,
                 timer: Callable | None = None, reset_to_zero: Sequence[str] = (),
                 restore_value: Sequence[str] = ()) -> None:
        if not configs:
            raise ValueError("autotune needs at least one config")
        unknown = [name for name in (*reset_to_zero, *restore_value) if name not in kernel.signature.parameters]
        if unknown:
            raise ValueError(f"reset_to_zero / restore_value name no parameter of the kernel: {unknown}")
        # Trials launch every config several times on the caller's buffers.  A kernel that
        # accumulates (tl.atomic_add) or works in place would see its own earlier trials: the
        # arrays named here are zeroed, or put back to what they held, before every trial
        # launch and once more after the last.
        self.reset_to_zero = tuple(reset_to_zero)
        self.restore_value = tuple(restore_value)
        self.kernel = kernel
        self.configs = list(configs)
        self.key_names = list(key)
        self.warmup, self.rep = warmup, rep
        self.timer = timer or device_timer
        self.cache: dict[tuple, Config] = {}
        self.timings: dict[tuple, dict[str, float]] = {}
        self.cache_path = Path(cache_path) if cache_path else None
        self.fn = kernel.fn
        self.signature = kernel.signature
        self._load_disk_cache()

    # -- persistence -------------------------------------------------------------

    def _load_disk_cache(self) -> None:
        if self.cache_path is None or not self.cache_path.exists():
            return
        try:
            stored = json.loads(self.cache_path.read_text())
        except (OSError, ValueError):
            return
        by_label = {config.label(): config for config in self.configs}
        for entry in stored.get(self.fn.__name__, []):
            config = by_label.get(entry.get("config"))
            # timings from another GPU model or another build of the runtime are not trusted
            if config is not None and entry.get("platform") == self._platform():
                self.cache[tuple(entry["key"])] = config

    def _save_disk_cache(self) -> None:
        if self.cache_path is None:
            return
        stored = {}
        if self.cache_path.exists():
            try:
                stored = json.loads(self.cache_path.read_text())
            except (OSError, ValueError):
                stored = {}
        stored[self.fn.__name__] = [
            {"key": list(key), "config": config.label(), "ms": self.timings.get(key, {}),
             "platform": self._platform()}
            for key, config in self.cache.items()
        ]
        self.cache_path.parent.mkdir(parents=True, exist_ok=True)
        # written beside the target and renamed into place, so that ranks saving at the same
        # time leave one complete file rather than an interleaved one
        scratch = self.cache_path.with_name(f"{self.cache_path.name}.{os.getpid()}.tmp")
        scratch.write_text(json.dumps(stored, indent=1))
        os.replace(scratch, self.cache_path)

    _platform_text: str | None = None

    def _platform(self) -> str:
        """GPU model and runtime-library version: what a stored timing is valid for."""
        if Autotuner._platform_text is None:
            from . import runtime

            try:
                gpu = runtime.device_info().name.decode(errors="replace") if runtime.is_available() else "no GPU"
            except Exception:
                gpu = "no GPU"
            try:
                version = runtime.library().mtb_version().decode(errors="replace")
            except Exception:
                version = "unknown runtime"
            Autotuner._platform_text = f"{gpu} / {version}"
        return Autotuner._platform_text

    # -- selection ---------------------------------------------------------------

    def _key(self, bound_arguments: dict[str, Any]) -> tuple:
        parts: list[Any] = [str(bound_arguments[name]) for name in self.key_names]
        for name, value in bound_arguments.items():
            info = arrays.describe(value)
            if info is not None:
                parts.append(f"{name}:{info.dtype}")
        return tuple(parts)

    def _on_device(self, arguments: dict[str, Any]) -> bool:
        infos = [info for info in map(arrays.describe, arguments.values()) if info is not None]
        return any(info.on_device for info in infos)

    def best_config(self, grid: Grid, args: tuple, kwargs: dict[str, Any]) -> Config:
        probe = {**self.configs[0].kwargs, **kwargs}
        bound = self.signature.bind(*args, **{k: v for k, v in probe.items() if k in self.signature.parameters})
        key = self._key(dict(bound.arguments))
        chosen = self.cache.get(key)
        if chosen is not None:
            return chosen
        if len(self.configs) == 1 or not self._on_device(dict(bound.arguments)):
            return self.configs[0]
        from .cuda_utils import current_stream

        results: dict[str, float] = {}
        best: tuple[float, Config] | None = None
        prepare = self._trial_reset(dict(bound.arguments))
        if prepare is None and self._accumulates(grid, args, kwargs):
            raise ValueError(
                f"{self.fn.__name__} accumulates into its arguments (tl.atomic_add): timing every config on "
                "the caller's buffers would add the trials up.  Name the accumulated arrays in "
                "reset_to_zero=[...] or restore_value=[...]")
        for config in self.configs:
            try:
                launch = self.kernel.launcher(grid, *args, **{**kwargs, **config.all_kwargs()})
                if prepare is None:
                    run = launch
                else:
                    def run(launch=launch) -> None:
                        prepare()
                        launch()
                ms = self.timer(run, current_stream, self.warmup, self.rep)
            except (TypeError, ValueError, RuntimeError) as error:
                results[config.label()] = float("inf")
                last_error = error
                continue
            results[config.label()] = ms
            if best is None or ms < best[0]:
                best = (ms, config)
        if prepare is not None:
            prepare()                         # the caller's own launch starts from clean buffers
            self._release_snapshots()
        if best is None:
            raise RuntimeError(f"no autotune config could be launched: {last_error}")
        self.cache[key] = best[1]
        self.timings[key] = results
        self._save_disk_cache()
        return best[1]

    def _accumulates(self, grid: Grid, args: tuple, kwargs: dict[str, Any]) -> bool:
        from .ssa import SSAForRange

        def has_atomic(ops) -> bool:
            return any(has_atomic(op.body) if isinstance(op, SSAForRange) else op.opcode == "atomic_add"
                       for op in ops)

        artifact = self.kernel._prepare(grid, args, {**kwargs, **self.configs[0].all_kwargs()})[0]
        return has_atomic(artifact.ssa_ops)

    def _trial_reset(self, arguments: dict[str, Any]):
        """A function that puts the named arrays back (zeros, or a snapshot taken now) on the
        current stream, or None when nothing was named."""
        if not self.reset_to_zero and not self.restore_value:
            return None
        from . import runtime
        from .cuda_utils import current_stream

        def span(name: str) -> tuple[int, int]:
            value = arguments[name]
            info = arrays.describe(value)
            if info is None or not info.on_device or not info.address:
                raise ValueError(f"{name} is not a device array")
            itemsize = {"float32": 4, "int32": 4, "bfloat16": 2, "float16": 2}.get(info.dtype, 1)
            return info.address, arrays.element_count(value) * itemsize

        zeroed = [span(name) for name in self.reset_to_zero]
        saved = []
        for name in self.restore_value:
            address, nbytes = span(name)
            copy = runtime.mem_alloc(max(nbytes, 16))
            runtime.memcpy_d2d(copy, address, nbytes, current_stream())
            saved.append((address, copy, nbytes))
        self._snapshots = saved               # freed when the tuning run is over

        def prepare() -> None:
            stream = current_stream()
            for address, nbytes in zeroed:
                runtime.memset_u32(address, 0, nbytes // 4, stream)
            for address, copy, nbytes in saved:
                runtime.memcpy_d2d(address, copy, nbytes, stream)

        return prepare

    def _release_snapshots(self) -> None:
        """Free the copies ``restore_value`` made, once the last restore has run."""
        from . import runtime
        from .cuda_utils import current_stream

        saved, self._snapshots = getattr(self, "_snapshots", []), []
        if saved:
            runtime.stream_synchronize(current_stream())
            for _, copy, _ in saved:
                runtime.mem_free(copy)

    # -- kernel protocol ---------------------------------------------------------

    def __getitem__(self, grid: Grid):
        def launch(*args, **kwargs):
            config = self.best_config(grid, args, kwargs)
            return self.kernel[grid](*args, **{**kwargs, **config.all_kwargs()})

        return launch

    def launcher(self, grid: Grid, *args, **kwargs):
        config = self.best_config(grid, args, kwargs)
        run = self.kernel.launcher(grid, *args, **{**kwargs, **config.all_kwargs()})
        run.config = config          # type: ignore[attr-defined]
        return run

    def clear_cache(self) -> None:
        self.cache.clear()
        self.timings.clear()
        self.kernel.clear_cache()


def autotune(configs: Sequence[Config], key: Sequence[str], warmup: int = 2, rep: int = 5,
             cache_path: str | os.PathLike | None = None, reset_to_zero: Sequence[str] = (),
             restore_value: Sequence[str] = ()):
    def decorate(kernel: CompiledKernel) -> Autotuner:
        if not isinstance(kernel, CompiledKernel):
            raise TypeError("@autotune goes above @jit")
        return Autotuner(kernel, configs, key, warmup, rep, cache_path, reset_to_zero=reset_to_zero,
                         restore_value=restore_value)

    return decorate
