"""Helpers for the GPU parity tests: seeded inputs, and three ways to run a case —
this backend, the reference's generated CUDA source (from the golden fixtures,
compiled with the reference's own NVRTC option and launch geometry), and the
CPU oracle."""

from __future__ import annotations

import ctypes
import zlib

import numpy as np

from mytriton_b200 import kernel_cases as cases
from mytriton_b200 import kernels as corpus
from mytriton_b200 import device, runtime
from mytriton_b200.cuda_utils import REFERENCE_NVRTC_OPTIONS

SPECIALS = np.array([np.nan, 0.0, -0.0, np.inf, -np.inf, 1.0, -1.0, 3.5], dtype=np.float32)


def seeded_arrays(case: cases.Case, specials: bool = False) -> list:
    """Host arguments for a case: arrays filled from a per-case seed, scalars as given."""
    rng = np.random.default_rng(zlib.crc32(case.name.encode()))
    out = []
    for arg in case.args:
        if isinstance(arg, tuple) and arg and arg[0] == "f32":
            data = rng.standard_normal(arg[1], dtype=np.float32)
            if specials and data.size >= SPECIALS.size:
                data.reshape(-1)[: SPECIALS.size] = SPECIALS
            out.append(data)
        else:
            out.append(arg)
    return out


def _to_device(host_args: list) -> list:
    return [device.to_device(a) if isinstance(a, np.ndarray) else a for a in host_args]


def _to_host(dev_args: list) -> list:
    return [a.to_host() if isinstance(a, device.DeviceArray) else a for a in dev_args]


def run_mine(case: cases.Case, host_args: list, **options) -> list:
    kernel = getattr(corpus, case.kernel)
    dev_args = _to_device(host_args)
    kernel[case.grid](*dev_args, **case.constexprs, **options)
    runtime.synchronize()
    return _to_host(dev_args)


_reference_modules: dict[str, runtime.Module] = {}


def run_reference_source(case: cases.Case, golden_entry: dict, host_args: list) -> list:
    """Compile and launch the CUDA text the reference generated for this case."""
    module = _reference_modules.get(case.name)
    if module is None:
        module = runtime.Module(golden_entry["cuda_src"], case.kernel, REFERENCE_NVRTC_OPTIONS)
        _reference_modules[case.name] = module
    dev_args = _to_device(host_args)
    packed = []
    for value in dev_args:
        if isinstance(value, device.DeviceArray):
            packed.append(ctypes.c_uint64(value.ptr))
        elif isinstance(value, (int, np.integer)):
            packed.append(ctypes.c_int32(int(value)))
        else:
            packed.append(ctypes.c_float(float(value)))
    module.launch(case.grid, (golden_entry["threads_per_block"],), packed)
    runtime.synchronize()
    return _to_host(dev_args)


def run_oracle(case: cases.Case, ssa_text: str, host_args: list) -> list:
    from oracle import ssa_interp

    kernel = getattr(corpus, case.kernel)
    names = [n for n in kernel.signature.parameters if n not in case.constexprs]
    copies = [a.copy() if isinstance(a, np.ndarray) else a for a in host_args]
    ssa_interp.run(ssa_text, dict(zip(names, copies)), case.grid)
    return copies


def same_bits(a: np.ndarray, b: np.ndarray) -> bool:
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


def same_values(a: np.ndarray, b: np.ndarray) -> bool:
    """Bit-identical wherever the value is not NaN, NaN in the same places.  (A GPU
    produces the canonical NaN 0x7fffffff where NumPy keeps the operand's payload,
    so NaN bit patterns are not comparable between a device and the host.)"""
    if a.shape != b.shape:
        return False
    nan_a, nan_b = np.isnan(a), np.isnan(b)
    if not np.array_equal(nan_a, nan_b):
        return False
    return np.array_equal(a.view(np.uint32)[~nan_a], b.view(np.uint32)[~nan_b])
