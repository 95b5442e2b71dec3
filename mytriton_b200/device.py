"""Minimal device arrays over the native runtime, for callers without torch.

``DeviceArray`` owns one allocation made through the C ABI
(``mtb_mem_alloc``) and exposes ``__cuda_array_interface__``, so it can be passed
to kernels exactly like a torch CUDA tensor.  It plays the part CuPy arrays play
in the reference's execution tests (``cp.asarray`` / ``cp.empty`` /
``cp.asnumpy``, e.g. ``tests/test_add_kernel.py:238-254``).
"""

from __future__ import annotations

import numpy as np

from . import runtime

_TYPESTR = {"float32": "<f4", "int32": "<i4", "bfloat16": "<u2", "float16": "<f2", "uint16": "<u2", "uint32": "<u4",
            "float8_e4m3fn": "|u1", "float8_e5m2": "|u1", "uint8": "|u1"}
_ITEMSIZE = {"float32": 4, "int32": 4, "bfloat16": 2, "float16": 2, "uint16": 2, "uint32": 4,
             "float8_e4m3fn": 1, "float8_e5m2": 1, "uint8": 1}


class DeviceArray:
    def __init__(self, shape, dtype: str = "float32", _borrowed_ptr: int | None = None) -> None:
        self.shape = tuple(int(d) for d in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        self.dtype_name = dtype
        self.itemsize = _ITEMSIZE[dtype]
        self.size = int(np.prod(self.shape)) if self.shape else 1
        self.nbytes = self.size * self.itemsize
        self.c_contiguous = True
        self.owns_memory = _borrowed_ptr is None
        self.ptr = runtime.mem_alloc(max(self.nbytes, 16)) if self.owns_memory else _borrowed_ptr

    def rows(self, start: int, stop: int) -> "DeviceArray":
        """A view of rows [start, stop) of a 2-D array.  The view does not own the
        memory: keep the parent alive while it is in use."""
        if len(self.shape) != 2 or not 0 <= start <= stop <= self.shape[0]:
            raise ValueError(f"bad row range [{start}, {stop}) for shape {self.shape}")
        offset = start * self.shape[1] * self.itemsize
        return DeviceArray((stop - start, self.shape[1]), self.dtype_name, _borrowed_ptr=self.ptr + offset)

    @property
    def __cuda_array_interface__(self) -> dict:
        return {
            "shape": self.shape,
            "typestr": _TYPESTR[self.dtype_name],
            "data": (self.ptr, False),
            "version": 3,
            "strides": None,
        }

    @property
    def ndim(self) -> int:
        return len(self.shape)

    # -- transfers (synchronous with respect to the given stream) -------------------

    def copy_from_host(self, host: np.ndarray, stream: int = 0) -> "DeviceArray":
        host = np.ascontiguousarray(host)
        if host.nbytes != self.nbytes:
            raise ValueError(f"size mismatch: host {host.nbytes} B, device {self.nbytes} B")
        if self.nbytes:
            runtime.memcpy_h2d(self.ptr, host.ctypes.data, self.nbytes, stream)
            runtime.stream_synchronize(stream)
        return self

    def to_host(self, stream: int = 0) -> np.ndarray:
        numpy_dtype = {"bfloat16": np.uint16, "float8_e4m3fn": np.uint8, "float8_e5m2": np.uint8}.get(self.dtype_name, self.dtype_name)
        host = np.empty(self.shape, dtype=numpy_dtype)
        if self.nbytes:
            runtime.memcpy_d2h(host.ctypes.data, self.ptr, self.nbytes, stream)
            runtime.stream_synchronize(stream)
        return host

    def fill_u32(self, pattern: int, stream: int = 0) -> "DeviceArray":
        runtime.memset_u32(self.ptr, pattern, self.nbytes // 4, stream)
        return self

    def free(self) -> None:
        if self.ptr and self.owns_memory:
            runtime.mem_free(self.ptr)
        self.ptr = 0

    def __del__(self) -> None:
        try:
            self.free()
        except Exception:
            pass


def to_device(host: np.ndarray, dtype: str | None = None) -> DeviceArray:
    """Copy a NumPy array to a new device array.  ``dtype="bfloat16"`` expects the
    16-bit patterns as uint16."""
    name = dtype or str(host.dtype)
    return DeviceArray(host.shape, name).copy_from_host(host)


def empty(shape, dtype: str = "float32") -> DeviceArray:
    return DeviceArray(shape, dtype)
