"""The debug bounds check: where out-of-range accesses are reported.

Kernels compiled with ``bounds_check=True`` compare every global load, store and atomic
with the extent of the array it addresses (the launcher passes the extents beside the
pointers).  An access outside the extent is *skipped* — a load yields zero, a store or an
atomic does nothing — and the first one is recorded in a per-device status block: which
parameter, which element index.  Nothing traps and the context stays usable; ``check()``
reads the record on the host.

The reference has no such mode (its Makefile runs no sanitizer either, ``Makefile:9-12``);
this is the stand-in for ``compute-sanitizer --tool memcheck`` on kernels this backend
generates.
"""

from __future__ import annotations

import ctypes

from . import runtime

_blocks: dict[int, int] = {}
_WORDS = 4


class OutOfBoundsError(RuntimeError):
    """A checked kernel made an access outside an array.  ``parameter`` is the position of
    the array among the kernel's run-time parameters, ``index`` the element index it used."""

    def __init__(self, parameter: int, index: int, name: str | None = None) -> None:
        self.parameter = parameter
        self.index = index
        self.name = name
        label = f"parameter #{parameter}" + (f" ({name})" if name else "")
        super().__init__(f"out-of-bounds access to {label} at element index {index} (the access was skipped)")


def status_block() -> int:
    """Device address of the current device's record (16 bytes, zero when clean)."""
    device = runtime.current_device()
    if device not in _blocks:
        pointer = runtime.mem_alloc(256)
        runtime.memset_u32(pointer, 0, 64)
        runtime.synchronize()
        _blocks[device] = pointer
    return _blocks[device]


def check(stream: int = 0, kernel=None) -> None:
    """Wait for ``stream`` and raise OutOfBoundsError if a checked kernel reported an access
    outside an array since the last call.  The record is cleared, so each report is raised
    once.  ``kernel`` (a jitted kernel) lets the message name the parameter."""
    device = runtime.current_device()
    if device not in _blocks:
        return
    words = (ctypes.c_uint32 * _WORDS)()
    runtime.memcpy_d2h(ctypes.addressof(words), _blocks[device], 4 * _WORDS, stream)
    runtime.stream_synchronize(stream)
    if words[0] == 0:
        return
    runtime.memset_u32(_blocks[device], 0, _WORDS, stream)
    runtime.stream_synchronize(stream)
    parameter = int(words[0] & 0x0FFFFFFF)
    index = int(words[1]) | (int(words[2]) << 32)
    if index >= 1 << 63:
        index -= 1 << 64
    name = None
    names = getattr(kernel, "_runtime_names", None)
    if names and parameter < len(names):
        name = names[parameter]
    raise OutOfBoundsError(parameter, index, name)
