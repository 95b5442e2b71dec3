"""Compile-and-launch glue between the JIT driver and the native runtime.

Keeps the contract of the reference's ``src/mytriton/cuda_utils.py:64-117``:

* host-only (NumPy) arguments mean *compile only* — nothing GPU-related is
  imported or initialised (``:94-96``);
* mixing host and device arrays is a ``TypeError`` (``:77-80``);
* ints are passed as 32-bit ints, floats as 32-bit floats (``:56-61``);
* launches are asynchronous and unchecked; the caller synchronises (``:113-117``).

CuPy is replaced by libmtb200.so (NVRTC + driver API, see runtime.py).  Device
arrays are ``torch`` CUDA tensors, ``DeviceArray`` objects from this package, or
anything with ``__cuda_array_interface__``.  There is no CPU execution path.
"""

from __future__ import annotations

import ctypes
import sys
from typing import Any

import numpy as np

from . import arrays
from .cuda_codegen import LaunchPlan

CudaKernelCache = dict[tuple[object, str], Any]

NVRTC_OPTIONS = ("--std=c++17",)
REFERENCE_NVRTC_OPTIONS = ("--std=c++14",)   # what the reference passes, cuda_utils.py:107-111


class CudaUnavailableError(RuntimeError):
    pass


def _runtime():
    from . import runtime

    return runtime


def _cupy():
    """The device runtime binding.  (The reference keeps its lazily imported CuPy module
    behind this name, src/mytriton/cuda_utils.py:23-27; code that patches it to prove that
    host-only calls never touch the GPU keeps working.)"""
    return _runtime()


def cuda_available() -> bool:
    try:
        return _runtime().is_available()
    except Exception:
        return False


def cuda_module():
    """The runtime binding, or CudaUnavailableError if no B200-class device answers."""
    runtime = _runtime()
    try:
        count = runtime.device_count()
    except runtime.RuntimeLibraryError as error:
        raise CudaUnavailableError(str(error)) from error
    if count <= 0:
        raise CudaUnavailableError("CUDA GPU is not available")
    return runtime


def cuda_execution_required(runtime_args: tuple[object, ...], *, backend_name: str) -> bool:
    infos = [info for info in map(arrays.describe, runtime_args) if info is not None]
    on_device = [info for info in infos if info.on_device]
    if not on_device:
        return False
    if len(on_device) != len(infos):
        raise TypeError(
            f"{backend_name} execution does not support mixed NumPy and CuPy arrays"
        )
    return True


def _current_stream_and_device(runtime_args: tuple[object, ...]) -> tuple[int, int | None]:
    """Launch on torch's current stream when the arguments are torch tensors."""
    for value in runtime_args:
        if type(value).__module__.startswith("torch") and hasattr(value, "data_ptr"):
            torch = sys.modules["torch"]
            device = value.device.index
            if device is None:
                device = torch.cuda.current_device()
            return int(torch.cuda.current_stream(device).cuda_stream), int(device)
        stream = getattr(value, "stream", None)
        if isinstance(stream, int):
            return stream, getattr(value, "device", None)
    return 0, None


def _marshal(value: object) -> ctypes._SimpleCData:
    info = arrays.describe(value)
    if info is not None:
        return ctypes.c_uint64(info.address or 0)
    if isinstance(value, (int, np.integer)):
        return ctypes.c_int32(int(value))
    if isinstance(value, (float, np.floating)):
        return ctypes.c_float(float(value))
    raise TypeError(f"unsupported kernel argument {type(value)}")


def _scalar(runtime_args, names, token: str) -> int:
    return int(token) if token.lstrip("-").isdigit() else int(runtime_args[names.index(token)])


def current_stream(device: int | None = None) -> int:
    """torch's current stream on ``device`` if torch is loaded, else the default stream."""
    torch = sys.modules.get("torch")
    if torch is None or not torch.cuda.is_initialized():
        return 0
    if device is None:
        device = torch.cuda.current_device()
    return int(torch._C._cuda_getCurrentRawStream(device))


def execute_cuda_if_needed(
    *,
    kernel_cache: CudaKernelCache,
    cuda_src: str,
    kernel_name: str,
    launch_grid: tuple[int, ...],
    threads_per_block: int,
    runtime_args: tuple[object, ...],
    plan: LaunchPlan | None = None,
    param_names: tuple[str, ...] = (),
    nvrtc_options: tuple[str, ...] = NVRTC_OPTIONS,
    prepare_only: bool = False,
    peer_stores: dict[str, list[int]] | None = None,
    extents: dict[str, int] | None = None,
):
    """Compile (cached) and launch.  With ``prepare_only`` nothing is launched: the
    return value is ``(prepared_launch, device)`` for repeated use, or None when the
    arguments are host arrays (compile-only)."""
    if not cuda_execution_required(runtime_args, backend_name="CUDA"):
        return None

    runtime = cuda_module()
    stream, device = _current_stream_and_device(runtime_args)
    previous = None
    if device is not None:
        # the arrays' device is made current for the compile-and-launch work below and the
        # caller's current device is put back afterwards
        previous = runtime.current_device()
        if previous == device:
            previous = None
        else:
            runtime.set_device(device)
    try:
        return _execute_on_current_device(
            runtime, stream, device, kernel_cache, cuda_src, kernel_name, launch_grid, threads_per_block,
            runtime_args, plan, param_names, nvrtc_options, prepare_only, peer_stores, extents)
    finally:
        if previous is not None:
            runtime.set_device(previous)


class _LaunchSequence:
    """Prepared launches that run one after the other on the stream given at call time."""

    def __init__(self, launches, keepalive) -> None:
        self.launches = launches
        self.keepalive = keepalive

    def __call__(self, stream: int = 0) -> None:
        for launch in self.launches:
            launch(stream)


def _launch_pair_of_kernels(runtime, stream, device, kernel_cache, nvrtc_options, prepare_only, first, user_args,
                            follow_up):
    module, grid, threads, args, smem, cluster = first
    key = (follow_up["src"], follow_up["name"])
    second = kernel_cache.get(key)
    if second is None:
        second = runtime.load_or_compile(follow_up["src"], follow_up["name"], nvrtc_options)
        kernel_cache[key] = second
    second_args = list(user_args) + list(follow_up["args"])
    if prepare_only:
        return _LaunchSequence(
            [module.prepare(grid, (threads,), args, dynamic_smem=smem, cluster=cluster),
             second.prepare(follow_up["grid"], (follow_up["threads"],), second_args)],
            follow_up["keepalive"]), device
    module.launch(grid, (threads,), args, dynamic_smem=smem, stream=stream, cluster=cluster)
    second.launch(follow_up["grid"], (follow_up["threads"],), second_args, stream=stream)
    # the workspace must outlive both kernels: freeing device memory waits for the work in flight
    runtime.stream_synchronize(stream)
    return None


def _execute_on_current_device(runtime, stream, device, kernel_cache, cuda_src, kernel_name, launch_grid,
                               threads_per_block, runtime_args, plan, param_names, nvrtc_options,
                               prepare_only, peer_stores, extents=None):
    info = runtime.device_info(device)
    if threads_per_block > info.max_threads_per_block:
        raise ValueError(
            f"CUDA block size {threads_per_block} exceeds device limit {info.max_threads_per_block}"
        )

    key = (cuda_src, kernel_name)
    module = kernel_cache.get(key)
    if module is None:
        module = runtime.load_or_compile(cuda_src, kernel_name, nvrtc_options)
        kernel_cache[key] = module

    args = [_marshal(value) for value in runtime_args]
    grid = tuple(launch_grid)
    smem = 0
    if plan is not None:
        smem = plan.dynamic_smem
        if plan.kind == "tcgen05":
            from . import dot_codegen

            grid, extra, follow_up = dot_codegen.prepare_launch(plan, runtime, info, launch_grid,
                                                                runtime_args, param_names, peer_stores)
            if follow_up is not None:
                # a split-K launch: a second kernel adds the partial sums up and stores C
                return _launch_pair_of_kernels(
                    runtime, stream, device, kernel_cache, nvrtc_options, prepare_only,
                    (module, grid, threads_per_block, args + extra, smem, plan.cluster), args, follow_up)
            args = args + extra
        elif peer_stores:
            raise ValueError("peer_stores applies to kernels lowered to the tcgen05 GEMM only")
        checked = plan.notes.get("bounds_check")
        if checked is not None:
            # kernels built with bounds_check=True take each array's extent (elements) and the
            # status block after their own parameters; `extents` narrows an array for this launch
            from . import bounds

            names = list(param_names)
            for name in checked:
                count = (extents or {}).get(name)
                if count is None:
                    count = arrays.element_count(runtime_args[names.index(name)])
                args.append(ctypes.c_int64(int(count)))
            args.append(ctypes.c_uint64(bounds.status_block()))
        elif extents:
            raise ValueError("extents applies to kernels compiled with bounds_check=True")
    cluster = plan.cluster if plan is not None else (1, 1, 1)
    if prepare_only:
        return module.prepare(grid, (threads_per_block,), args, dynamic_smem=smem, cluster=cluster), device
    module.launch(grid, (threads_per_block,), args, dynamic_smem=smem, stream=stream, cluster=cluster)
    return None
