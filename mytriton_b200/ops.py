"""Library operations backed by ahead-of-time compiled kernels in libmtb200.so.

``long_row_sum`` is the multi-CTA row sum the kernel language cannot express
(one program per row): rows are split over several CTAs and combined in a fixed
order, so a matrix with few, very long rows still fills the GPU.
"""

from __future__ import annotations

import ctypes as C

from . import arrays, runtime
from .cuda_utils import current_stream


def _device_f32(name: str, value) -> int:
    info = arrays.describe(value)
    if info is None or not info.on_device:
        raise TypeError(f"{name}: expected a device array")
    if info.dtype != "float32" or not info.contiguous:
        raise TypeError(f"{name}: expected a C-contiguous float32 array")
    return int(info.address)


def long_row_sum_scratch_bytes(rows: int, cols: int) -> int:
    size = C.c_size_t()
    runtime.call("mtb_long_row_sum_scratch_bytes", rows, cols, C.byref(size))
    return size.value


def long_row_sum(x, out, rows: int, cols: int, scratch, scratch_bytes: int,
                 stream: int | None = None) -> None:
    """out[r] = sum(x[r, :]) for a [rows, cols] fp32 matrix; asynchronous.

    ``scratch`` is a device array (or raw device address) of at least
    ``long_row_sum_scratch_bytes(rows, cols)`` bytes, owned by the caller."""
    scratch_ptr = scratch if isinstance(scratch, int) else int(arrays.describe(scratch).address)
    runtime.call(
        "mtb_long_row_sum", C.c_uint64(_device_f32("x", x)), C.c_uint64(_device_f32("out", out)),
        rows, cols, C.c_uint64(scratch_ptr), scratch_bytes,
        C.c_void_p(current_stream() if stream is None else stream))


def long_row_sum_static(x, out, rows: int, cols: int, stream: int | None = None) -> None:
    """``long_row_sum`` without a scratch argument, for callers that must not allocate.

    The partial sums go to a fixed block of device memory built into the library, so
    nothing is allocated or freed — useful once a process has handed all device memory
    to its own pool, or inside a loop that cannot tolerate an allocation's stall.
    At most 4096 rows and ``rows * splits <= 16384``; larger problems raise
    ``RuntimeLibraryError`` (code -7).  Call it once during set-up on each device
    (the first call resolves the block's address) and before starting any stream
    capture.  Calls share the block: do not let two of them overlap on one GPU."""
    runtime.call(
        "mtb_long_row_sum_static", C.c_uint64(_device_f32("x", x)),
        C.c_uint64(_device_f32("out", out)), rows, cols,
        C.c_void_p(current_stream() if stream is None else stream))

