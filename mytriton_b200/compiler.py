"""``@jit`` kernels: argument binding, specialisation cache, compile pipeline, launch.

The call protocol is the reference's (``src/mytriton/compiler.py:89-221``):
``kernel[grid](*args, **constexprs)`` binds arguments, evaluates the grid (an
int, a 1-3 sequence of positive ints, or a callable of the constexpr ``meta``
dict), specialises on runtime argument *types* and constexpr *values*, compiles
on a cache miss (trace -> SSA -> verify -> optimise -> verify -> CUDA), launches
when the arrays live on a GPU, and returns independent copies of
``(ops, ssa_ops, cuda_source)``.

Additions: the backend knobs ``num_warps``, ``num_stages`` and
``online_softmax`` may be passed as extra keyword arguments at launch (they are
part of the cache key, not of the kernel signature), and ``launcher(grid, ...)``
returns a pre-bound callable for hot loops that skips the per-call copy of the IR.
"""

from __future__ import annotations

import inspect
import os
import pickle
from collections.abc import Callable, Sequence
from copy import deepcopy
from dataclasses import dataclass
from typing import Any, Generic, ParamSpec, TypeAlias

from .ast_frontend import trace
from .cuda_codegen import LaunchPlan, SSACUDACodegen
from .cuda_utils import CudaKernelCache, current_stream, execute_cuda_if_needed
from .optim import ConstantFoldPass, CSEPass, DCEPass, PassManager, codegen_pipeline
from .ssa import SSAForRange, SSAItem, SSALowering
from .ssa_verification import SSAVerifier
from . import arrays
from .trace import Param, _make_param, is_constexpr_annotation

P = ParamSpec("P")
Meta: TypeAlias = dict[str, Any]
LaunchDimensions: TypeAlias = int | Sequence[int]
Grid: TypeAlias = LaunchDimensions | Callable[[Meta], LaunchDimensions]
CompilationResult: TypeAlias = tuple[list[Any], list[SSAItem], str]

BACKEND_OPTIONS = ("num_warps", "num_stages", "online_softmax", "elems_per_thread", "cta_group",
                   "min_ctas_per_sm", "group_m", "tensor_cores", "a_rows", "loop_passes", "cta_rows", "bounds_check",
                   "tile_n", "split_k")
LAUNCH_OPTIONS = ("peer_stores", "extents")      # affect one launch, not the generated code


def _constexpr_key(meta: dict[str, object]) -> tuple[tuple[str, type[object], object], ...]:
    entries = []
    for name, value in meta.items():
        if not isinstance(value, (bool, int, float, str)):
            raise TypeError(f"{name}: constexpr value must be bool, int, float, or str")
        entries.append((name, type(value), float(value).hex() if isinstance(value, float) else value))
    return tuple(entries)


@dataclass(frozen=True)
class _CompilationArtifact:
    ops: tuple[Any, ...]
    ssa_ops: tuple[SSAItem, ...]
    src: str
    threads_per_block: int
    plan: LaunchPlan
    frozen_ir: bytes | None   # pickled (ops, ssa_ops): cheaper to revive than deepcopy


class _LazyResult(tuple):
    """``(ops, ssa_ops, cuda_source)`` whose IR copies are made on first access.

    Callers get independent copies of the cached IR, as the reference promises
    (``src/mytriton/compiler.py:215-219``), but a caller that ignores the return
    value — every launch in a hot loop — does not pay for reviving them."""

    def __new__(cls, artifact: "_CompilationArtifact"):
        self = super().__new__(cls, (None, None, artifact.src))
        self._artifact = artifact
        self._items = None
        return self

    def _materialise(self) -> tuple:
        if self._items is None:
            artifact = self._artifact
            if artifact.frozen_ir is not None:
                ops, ssa_ops = pickle.loads(artifact.frozen_ir)
            else:
                ops, ssa_ops = deepcopy(artifact.ops), deepcopy(artifact.ssa_ops)
            self._items = (list(ops), list(ssa_ops), artifact.src)
        return self._items

    def __iter__(self):
        return iter(self._materialise())

    def __getitem__(self, index):
        return self._materialise()[index]

    def __len__(self) -> int:
        return 3

    def __eq__(self, other) -> bool:
        return self._materialise() == other

    def __ne__(self, other) -> bool:
        return not self == other

    __hash__ = None

    def __repr__(self) -> str:
        return repr(self._materialise())


def _normalise_grid(grid: Grid, meta: Meta) -> tuple[int, ...]:
    dims = grid(meta) if callable(grid) else grid
    if isinstance(dims, int):
        dims = (dims,)
    dims = tuple(dims)
    if not 1 <= len(dims) <= 3 or any(type(d) is not int or d <= 0 for d in dims):
        raise ValueError(f"invalid launch grid: {dims}")
    return dims


class CompiledKernel(Generic[P]):
    def __init__(self, fn: Callable[P, Any]) -> None:
        self.fn = fn
        signature = inspect.signature(fn)
        hints = inspect.get_annotations(fn, eval_str=True)
        self.signature = signature.replace(
            parameters=[
                p.replace(annotation=hints.get(name, p.annotation))
                for name, p in signature.parameters.items()
            ]
        )
        self._constexpr_names = tuple(
            name for name, p in self.signature.parameters.items()
            if is_constexpr_annotation(p.annotation)
        )
        self._runtime_names = tuple(
            name for name in self.signature.parameters if name not in self._constexpr_names
        )
        # Kernels that use tl.dot get Triton's own specialisation of integer arguments equal to 1
        # (they are folded into the IR as the constant), so that a matmul written with stride
        # arguments — `a + offs_m[:, None] * stride_am + offs_k[None, :] * stride_ak` — shows the
        # loop matcher which stride is the unit one.  Other kernels are traced as the reference
        # traces them, whatever their arguments.
        try:
            self._specialise_ones = ".dot(" in inspect.getsource(fn)
        except (OSError, TypeError):
            self._specialise_ones = False
        self.compilation_cache: dict[tuple[object, ...], _CompilationArtifact] = {}
        self.cuda_cache: CudaKernelCache = {}
        self._prepared: dict[tuple, Any] = {}
        self._last_infos: tuple = ()

    def clear_cache(self) -> None:
        self.compilation_cache.clear()
        self.cuda_cache.clear()
        self._prepared.clear()

    def _resolve_backend(self) -> str:
        selected = os.environ.get("MYTRITON_BACKEND", "cuda")
        if selected == "mlir":
            raise ValueError("the MLIR backend is not part of this build; only 'cuda' (sm_100a)")
        if selected != "cuda":
            raise ValueError(f"unsupported backend {selected!r}; expected 'cuda' or 'mlir'")
        return selected

    # -- compile -----------------------------------------------------------------

    def _split_options(self, kwargs: dict[str, Any]) -> dict[str, Any]:
        return {
            name: kwargs.pop(name)
            for name in BACKEND_OPTIONS
            if name in kwargs and name not in self.signature.parameters
        }

    def _compile(self, bound, params, options: dict[str, Any], ones: tuple[str, ...] = ()) -> _CompilationArtifact:
        ops, params = trace(self.fn, self.signature, bound.arguments, runtime_params=params,
                            constants=dict.fromkeys(ones, 1))
        ssa_ops = SSALowering().lower(ops)
        verifier = SSAVerifier(None)
        verifier.verify(ssa_ops)
        passes = [ConstantFoldPass(), CSEPass(), DCEPass()]
        ssa_ops = PassManager(passes, verifier).run(ssa_ops)
        # What callers get back is the reference's SSA (no passes once a run-time loop is
        # present).  The code generator consumes a further optimised copy: passes that work
        # inside loop bodies plus loop-invariant motion, unless ``loop_passes=False``.
        codegen_ops = ssa_ops
        if options.get("loop_passes", True) and any(isinstance(op, SSAForRange) for op in ssa_ops):
            codegen_ops = codegen_pipeline(verifier).run(list(ssa_ops))
        backend_options = {name: value for name, value in options.items() if name != "loop_passes"}
        artifact = SSACUDACodegen(**backend_options).generate_artifact(self.fn.__name__, codegen_ops, params)
        try:
            frozen = pickle.dumps((ops, ssa_ops), protocol=pickle.HIGHEST_PROTOCOL)
        except Exception:
            frozen = None
        return _CompilationArtifact(
            tuple(ops), tuple(ssa_ops), artifact.src, artifact.plan.threads, artifact.plan, frozen
        )

    def _prepare(self, grid: Grid, args, kwargs):
        kwargs = dict(kwargs)
        options = self._split_options(kwargs)
        launch_options = {
            name: kwargs.pop(name) for name in LAUNCH_OPTIONS
            if name in kwargs and name not in self.signature.parameters
        }
        bound = self.signature.bind(*args, **kwargs)
        bound.apply_defaults()
        meta: Meta = {name: bound.arguments[name] for name in self._constexpr_names}
        launch_grid = _normalise_grid(grid, meta)
        runtime_args = tuple(bound.arguments[name] for name in self._runtime_names)
        infos = tuple(arrays.describe(value) for value in runtime_args)
        params: list[Param] = [
            _make_param(name, value, info)
            for name, value, info in zip(self._runtime_names, runtime_args, infos)
        ]
        backend = self._resolve_backend()
        ones = tuple(name for name, value in zip(self._runtime_names, runtime_args)
                     if type(value) is int and value == 1) if self._specialise_ones else ()
        key = (
            backend, ones, tuple(param.ty for param in params), _constexpr_key(meta),
            tuple(sorted(options.items())),
        )
        artifact = self.compilation_cache.get(key)
        if artifact is None:
            artifact = self._compile(bound, params, options, ones)
            self.compilation_cache[key] = artifact
        if artifact.plan.kind == "tcgen05" and not launch_options \
                and any(info is not None and info.on_device for info in infos):
            # operands TMA cannot address (odd row strides, unaligned bases) or a third grid
            # axis: this launch uses the kernel's SIMT variant, compiled on first need
            from . import dot_codegen

            obstacle = dot_codegen.launch_obstacle(artifact.plan, launch_grid, runtime_args, self._runtime_names)
            if obstacle:
                simt_key = key[:-1] + (tuple(sorted({**options, "tensor_cores": False}.items())),)
                artifact = self.compilation_cache.get(simt_key)
                if artifact is None:
                    try:
                        artifact = self._compile(bound, params, {**options, "tensor_cores": False}, ones)
                    except TypeError as error:
                        raise dot_codegen.GemmLaunchError(f"{obstacle}; no SIMT variant either: {error}") from error
                    self.compilation_cache[simt_key] = artifact
        if artifact.plan.kind == "tcgen05" and not launch_options and not options.keys() & {
                "cta_group", "num_stages", "a_rows", "group_m", "cta_rows", "tile_n", "split_k"} \
                and any(info is not None and info.on_device for info in infos):
            # a launch that covers only a few rows of C: the variant that fetches just those rows
            # of A, in narrow deep tiles, streams B faster (compiled on first need)
            from . import dot_codegen

            skinny = dot_codegen.skinny_launch_options(artifact.plan, launch_grid, runtime_args, self._runtime_names)
            if skinny is not None:
                skinny_options = {**options, **skinny}
                skinny_key = key[:-1] + (tuple(sorted(skinny_options.items())),)
                artifact = self.compilation_cache.get(skinny_key)
                if artifact is None:
                    artifact = self._compile(bound, params, skinny_options, ones)
                    self.compilation_cache[skinny_key] = artifact
        if artifact.plan.kind == "tcgen05" and not launch_options and not options.keys() & {
                "cta_group", "num_stages", "a_rows", "group_m", "cta_rows", "tile_n", "split_k"} \
                and any(info is not None and info.on_device for info in infos):
            # too few tiles to fill the GPU with CTA pairs: single CTAs on narrower tiles, several
            # units of work per tile along a deep K (compiled on first need)
            from . import dot_codegen

            small = dot_codegen.prefers_small_problem_variant(
                artifact.plan, launch_grid, runtime_args, self._runtime_names)
            if small:
                small_options = {**options, **small}
                small_key = key[:-1] + (tuple(sorted(small_options.items())),)
                artifact = self.compilation_cache.get(small_key)
                if artifact is None:
                    artifact = self._compile(bound, params, small_options, ones)
                    self.compilation_cache[small_key] = artifact
        if artifact.plan.kind == "tcgen05" and artifact.plan.notes.get("cta_rows") == 256 \
                and not launch_options and "cta_rows" not in options \
                and any(info is not None and info.on_device for info in infos):
            # too few 512-row tiles for the GPU's CTA pairs: this launch uses the 256-row tiling
            from . import dot_codegen

            if dot_codegen.prefers_narrow_tiles(artifact.plan, launch_grid, runtime_args, self._runtime_names):
                narrow_options = {**options, "cta_rows": 128}
                narrow_key = key[:-1] + (tuple(sorted(narrow_options.items())),)
                artifact = self.compilation_cache.get(narrow_key)
                if artifact is None:
                    artifact = self._compile(bound, params, narrow_options, ones)
                    self.compilation_cache[narrow_key] = artifact
        self._last_infos = infos
        return artifact, launch_grid, runtime_args, launch_options

    def _launch_cached(self, artifact, launch_grid, runtime_args, infos) -> None:
        """Launch through a prepared launch remembered per (kernel variant, grid,
        argument addresses and scalar values): a repeat call costs one C call."""
        if not any(info is not None and info.on_device for info in infos):
            return                                   # host arrays only: compile-only call
        key = (id(artifact), launch_grid, tuple(
            (type(value), value) if info is None else info.address
            for value, info in zip(runtime_args, infos)))
        prepared = self._prepared.get(key)
        if prepared is None:
            prepared = self._execute(artifact, launch_grid, runtime_args, prepare_only=True)
            if len(self._prepared) >= 256:
                self._prepared.clear()
            self._prepared[key] = prepared
        launch, device = prepared
        launch(current_stream(device))

    def _execute(self, artifact: _CompilationArtifact, launch_grid, runtime_args,
                 launch_options=None, prepare_only=False):
        return execute_cuda_if_needed(
            kernel_cache=self.cuda_cache,
            cuda_src=artifact.src,
            kernel_name=self.fn.__name__,
            launch_grid=launch_grid,
            threads_per_block=artifact.threads_per_block,
            runtime_args=runtime_args,
            plan=artifact.plan,
            param_names=self._runtime_names,
            prepare_only=prepare_only,
            **(launch_options or {}),
        )

    # -- public ------------------------------------------------------------------

    def __getitem__(self, grid: Grid) -> Callable[P, CompilationResult]:
        def launch(*args: P.args, **kwargs: P.kwargs) -> CompilationResult:
            artifact, launch_grid, runtime_args, launch_options = self._prepare(grid, args, kwargs)
            if launch_options:
                self._execute(artifact, launch_grid, runtime_args, launch_options)
            else:
                self._launch_cached(artifact, launch_grid, runtime_args, self._last_infos)
            return _LazyResult(artifact)

        return launch

    def launcher(self, grid: Grid, *args, **kwargs) -> Callable[[], None]:
        """Compile for these arguments once and return ``run()`` that only launches.

        Pointers and scalars are captured now: ``run()`` re-launches on the same
        buffers (their contents may change, their addresses must not) with a single
        C call, on torch's current stream when torch is in use.  With host (NumPy)
        arguments ``run()`` does nothing, like the compile-only call."""
        artifact, launch_grid, runtime_args, launch_options = self._prepare(grid, args, kwargs)
        prepared = self._execute(artifact, launch_grid, runtime_args, launch_options, prepare_only=True)
        if prepared is None:
            def run() -> None:
                return None
        else:
            launch, device = prepared

            def run() -> None:
                launch(current_stream(device))
        run.keepalive = runtime_args     # type: ignore[attr-defined]

        run.artifact = artifact          # type: ignore[attr-defined]
        run.grid = launch_grid           # type: ignore[attr-defined]
        return run


def jit(fn: Callable[P, Any]) -> CompiledKernel[P]:
    return CompiledKernel(fn)
