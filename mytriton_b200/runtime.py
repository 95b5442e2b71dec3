"""ctypes binding of libmtb200.so (the C ABI in include/mtb200_rt.h).

This is the only place that talks to the GPU.  There is no fallback: if the
library is missing or the driver cannot be initialised, the calls raise.
Compiling (NVRTC) works without a GPU; loading and launching do not.
"""

from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path
from typing import Sequence

LIBRARY_PATH = Path(__file__).resolve().parent / "libmtb200.so"
ARCH = "sm_100a"


class RuntimeLibraryError(RuntimeError):
    """A C-ABI call returned non-zero."""

    def __init__(self, function: str, code: int, message: str) -> None:
        super().__init__(f"{function} failed ({code}): {message}")
        self.function = function
        self.code = code


class DeviceInfo(C.Structure):
    _fields_ = [
        ("name", C.c_char * 128),
        ("cc_major", C.c_int), ("cc_minor", C.c_int),
        ("sm_count", C.c_int),
        ("max_threads_per_block", C.c_int),
        ("max_smem_per_block_optin", C.c_int),
        ("l2_bytes", C.c_int),
        ("sm_clock_khz", C.c_int), ("mem_clock_khz", C.c_int),
        ("total_mem_bytes", C.c_uint64),
    ]


_u3 = C.c_uint * 3
_PROTOTYPES = {
    "mtb_init": [],
    "mtb_device_count": [C.POINTER(C.c_int)],
    "mtb_device_set": [C.c_int],
    "mtb_device_get": [C.POINTER(C.c_int)],
    "mtb_device_info": [C.c_int, C.POINTER(DeviceInfo)],
    "mtb_device_sync": [],
    "mtb_mem_info": [C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)],
    "mtb_compile": [C.c_char_p, C.c_char_p, C.c_char_p, C.POINTER(C.c_char_p), C.c_int,
                    C.POINTER(C.c_void_p), C.c_char_p, C.c_size_t],
    "mtb_module_cubin": [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)],
    "mtb_module_from_cubin": [C.c_void_p, C.c_size_t, C.c_char_p, C.POINTER(C.c_void_p)],
    "mtb_module_load": [C.c_void_p, C.c_int],
    "mtb_module_attr": [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int),
                        C.POINTER(C.c_int), C.POINTER(C.c_int)],
    "mtb_module_free": [C.c_void_p],
    "mtb_launch": [C.c_void_p, _u3, _u3, _u3, C.c_uint, C.c_void_p, C.POINTER(C.c_void_p)],
    "mtb_launch_on_device": [C.c_void_p, C.c_int, _u3, _u3, _u3, C.c_uint, C.c_void_p, C.POINTER(C.c_void_p)],
    "mtb_tensormap_encode_2d": [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_uint64, C.c_uint64,
                                C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.c_int, C.c_int],
    "mtb_stream_create": [C.POINTER(C.c_void_p)],
    "mtb_stream_destroy": [C.c_void_p],
    "mtb_stream_sync": [C.c_void_p],
    "mtb_event_create": [C.POINTER(C.c_void_p)],
    "mtb_event_destroy": [C.c_void_p],
    "mtb_event_record": [C.c_void_p, C.c_void_p],
    "mtb_event_sync": [C.c_void_p],
    "mtb_event_elapsed_ms": [C.c_void_p, C.c_void_p, C.POINTER(C.c_float)],
    "mtb_mem_alloc": [C.POINTER(C.c_uint64), C.c_size_t],
    "mtb_mem_free": [C.c_uint64],
    "mtb_memcpy_h2d": [C.c_uint64, C.c_void_p, C.c_size_t, C.c_void_p],
    "mtb_memcpy_d2h": [C.c_void_p, C.c_uint64, C.c_size_t, C.c_void_p],
    "mtb_memcpy_d2d": [C.c_uint64, C.c_uint64, C.c_size_t, C.c_void_p],
    "mtb_memset_u32": [C.c_uint64, C.c_uint32, C.c_size_t, C.c_void_p],
    "mtb_host_alloc_pinned": [C.POINTER(C.c_void_p), C.c_size_t],
    "mtb_host_free_pinned": [C.c_void_p],
    "mtb_status_check": [C.c_uint64, C.c_void_p, C.POINTER(C.c_uint32)],
    "mtb_long_row_sum_scratch_bytes": [C.c_int, C.c_longlong, C.POINTER(C.c_size_t)],
    "mtb_long_row_sum": [C.c_uint64, C.c_uint64, C.c_int, C.c_longlong, C.c_uint64, C.c_size_t,
                         C.c_void_p],
    "mtb_long_row_sum_static": [C.c_uint64, C.c_uint64, C.c_int, C.c_longlong, C.c_void_p],
}
EXPORTED_SYMBOLS = (*_PROTOTYPES, "mtb_last_error", "mtb_version", "mtb_set_last_error")

_lock = threading.Lock()
_lib: C.CDLL | None = None


def library() -> C.CDLL:
    """Load libmtb200.so (once) and declare every prototype."""
    global _lib
    with _lock:
        if _lib is None:
            if not LIBRARY_PATH.exists():
                raise RuntimeLibraryError(
                    "dlopen", -1,
                    f"{LIBRARY_PATH} is missing; build it with "
                    "`python -m mytriton_b200.build` (there is no CPU fallback)",
                )
            lib = C.CDLL(str(LIBRARY_PATH))
            for name, argtypes in _PROTOTYPES.items():
                fn = getattr(lib, name)
                fn.argtypes = argtypes
                fn.restype = C.c_int
            lib.mtb_last_error.restype = C.c_char_p
            lib.mtb_version.restype = C.c_char_p
            _lib = lib
        return _lib


def call(name: str, *args) -> None:
    lib = library()
    code = getattr(lib, name)(*args)
    if code != 0:
        raise RuntimeLibraryError(name, code, lib.mtb_last_error().decode(errors="replace"))


# ------------------------------------------------------------------ devices

def init() -> None:
    call("mtb_init")


def device_count() -> int:
    n = C.c_int(0)
    call("mtb_device_count", C.byref(n))
    return n.value


def is_available() -> bool:
    try:
        return device_count() > 0
    except (RuntimeLibraryError, OSError):
        return False


def set_device(index: int) -> None:
    call("mtb_device_set", index)


def current_device() -> int:
    n = C.c_int(0)
    call("mtb_device_get", C.byref(n))
    return n.value


_info_cache: dict[int, DeviceInfo] = {}


def device_info(index: int | None = None) -> DeviceInfo:
    index = current_device() if index is None else index
    if index not in _info_cache:
        info = DeviceInfo()
        call("mtb_device_info", index, C.byref(info))
        _info_cache[index] = info
    return _info_cache[index]


def synchronize() -> None:
    call("mtb_device_sync")


def mem_info() -> tuple[int, int]:
    free, total = C.c_uint64(0), C.c_uint64(0)
    call("mtb_mem_info", C.byref(free), C.byref(total))
    return free.value, total.value


# ------------------------------------------------------------------ modules

class Module:
    """One compiled kernel: cubin from NVRTC, loaded lazily on each device it is launched on
    (the native module keeps one loaded image per device)."""

    def __init__(self, source: str | None, name: str, options: Sequence[str] = (), arch: str = ARCH,
                 cubin: bytes | None = None):
        self.name = name
        self.handle = C.c_void_p()
        self.loaded_smem: dict[int, int] = {}      # device -> dynamic shared memory it was loaded for
        self.log = ""
        if cubin is not None:                      # revive a cached binary: no NVRTC involved
            call("mtb_module_from_cubin", cubin, len(cubin), name.encode(), C.byref(self.handle))
            return
        log = C.create_string_buffer(16384)
        opts = (C.c_char_p * max(1, len(options)))(*[o.encode() for o in options])
        try:
            call("mtb_compile", source.encode(), name.encode(), arch.encode(), opts,
                 len(options), C.byref(self.handle), log, len(log))
        finally:
            self.log = log.value.decode(errors="replace")

    def cubin(self) -> bytes:
        data, size = C.c_void_p(), C.c_size_t()
        call("mtb_module_cubin", self.handle, C.byref(data), C.byref(size))
        return C.string_at(data.value, size.value)

    def load(self, dynamic_smem: int = 0) -> "Module":
        """Load on the current device (once per device; again if more dynamic shared memory
        is asked for than it was loaded with)."""
        device = current_device()
        if dynamic_smem > self.loaded_smem.get(device, -1):
            call("mtb_module_load", self.handle, dynamic_smem)
            self.loaded_smem[device] = dynamic_smem
        return self

    def attributes(self) -> dict[str, int]:
        regs, smem, local, threads = (C.c_int() for _ in range(4))
        call("mtb_module_attr", self.handle, C.byref(regs), C.byref(smem), C.byref(local),
             C.byref(threads))
        return {"registers": regs.value, "static_smem": smem.value,
                "local_bytes": local.value, "max_threads": threads.value}

    def launch(self, grid, block, args: Sequence[C._SimpleCData | C.Structure | C.Array],
               dynamic_smem: int = 0, stream: int = 0, cluster=(1, 1, 1)) -> None:
        """Asynchronous launch.  ``args`` are ctypes objects, one per kernel parameter."""
        self.load(dynamic_smem)
        pointers = (C.c_void_p * max(1, len(args)))(
            *[C.cast(C.byref(a), C.c_void_p) for a in args]
        )
        call("mtb_launch", self.handle, _u3(*_pad3(grid)), _u3(*_pad3(block)),
             _u3(*_pad3(cluster)), dynamic_smem, C.c_void_p(stream), pointers)

    def prepare(self, grid, block, args, dynamic_smem: int = 0, cluster=(1, 1, 1)) -> "PreparedLaunch":
        """Bind everything but the stream once; the result re-launches with one C call, on the
        device that is current now (whatever device is current when it is called)."""
        self.load(dynamic_smem)
        return PreparedLaunch(self, grid, block, args, dynamic_smem, cluster, current_device())

    def __del__(self) -> None:
        handle, self.handle = getattr(self, "handle", None), None
        if handle and _lib is not None:
            try:
                _lib.mtb_module_free(handle)
            except Exception:  # interpreter shutdown
                pass


class PreparedLaunch:
    """A launch with its arguments already marshalled (hot loops, benchmarks)."""

    def __init__(self, module: Module, grid, block, args, dynamic_smem: int, cluster, device: int) -> None:
        self.module = module                      # keeps the module alive
        self.device = device                      # the pointers in `args` belong to this device
        self.args = list(args)                    # keeps the ctypes values alive
        self._grid, self._block = _u3(*_pad3(grid)), _u3(*_pad3(block))
        self._cluster = _u3(*_pad3(cluster))
        self._smem = dynamic_smem
        self._pointers = (C.c_void_p * max(1, len(self.args)))(
            *[C.cast(C.byref(a), C.c_void_p) for a in self.args]
        )
        self._launch = library().mtb_launch_on_device
        self._handle = module.handle

    def __call__(self, stream: int = 0) -> None:
        code = self._launch(self._handle, self.device, self._grid, self._block, self._cluster, self._smem,
                            stream, self._pointers)
        if code != 0:
            raise RuntimeLibraryError("mtb_launch", code,
                                      library().mtb_last_error().decode(errors="replace"))


def cache_directory() -> Path | None:
    """Where compiled kernels are kept between processes, or None if disabled.

    ``MYTRITON_B200_CACHE`` names the directory; ``MYTRITON_B200_CACHE=0`` (or empty)
    turns the cache off.  Default: ``~/.cache/mytriton_b200``."""
    import os

    chosen = os.environ.get("MYTRITON_B200_CACHE")
    if chosen is not None:
        return Path(chosen) if chosen not in ("", "0") else None
    return Path.home() / ".cache" / "mytriton_b200"


def load_or_compile(source: str, name: str, options: Sequence[str] = (), arch: str = ARCH) -> Module:
    """A Module for ``source``, from the on-disk cubin cache when it holds one.

    The key covers the source text, kernel name, NVRTC options, target and this
    library's version string; entries are written atomically, and a cache that cannot
    be read or written is simply bypassed."""
    import hashlib
    import os

    directory = cache_directory()
    if directory is None:
        return Module(source, name, options, arch)
    version = library().mtb_version()
    digest = hashlib.sha256(
        b"\0".join([source.encode(), name.encode(), arch.encode(), version,
                    *[o.encode() for o in options]])).hexdigest()
    path = directory / f"{name}-{digest[:32]}.cubin"
    try:
        return Module(None, name, cubin=path.read_bytes())
    except (OSError, RuntimeLibraryError):
        pass
    module = Module(source, name, options, arch)
    try:
        directory.mkdir(parents=True, exist_ok=True)
        scratch = path.with_suffix(f".{os.getpid()}.tmp")
        scratch.write_bytes(module.cubin())
        os.replace(scratch, path)
    except OSError:
        pass
    return module


def _pad3(dims) -> tuple[int, int, int]:
    dims = tuple(int(d) for d in dims)
    return (dims + (1, 1, 1))[:3]


# ------------------------------------------------------------------ tensor maps

class TensorMap(C.Structure):
    """128-byte CUtensorMap, passed by value as a ``__grid_constant__`` parameter."""

    _fields_ = [("opaque", C.c_uint64 * 16)]


class TensorMaps8(C.Structure):
    """Eight tensor maps in one by-value kernel parameter (output fan-out)."""

    _fields_ = [("m", TensorMap * 8)]


SWIZZLE_NONE, SWIZZLE_32B, SWIZZLE_64B, SWIZZLE_128B = 0, 1, 2, 3
SWIZZLE_128B_ATOM_32B = 4          # 128-byte span swizzled in 32-byte chunks (4-byte N-major operands)


def aligned_struct(kind):
    """A zeroed instance of ``kind`` at a 64-byte aligned address (ctypes alone does
    not honour that alignment, which cuTensorMapEncodeTiled requires)."""
    raw = C.create_string_buffer(C.sizeof(kind) + 64)
    address = (C.addressof(raw) + 63) & ~63
    instance = kind.from_address(address)
    instance._keepalive = raw
    return instance


def encode_tensormap_2d(base: int, dim_inner: int, dim_outer: int, stride_outer_bytes: int,
                        box_inner: int, box_outer: int, *, elem_bytes: int = 2,
                        is_float: bool = True, is_bf16: bool = True,
                        swizzle: int = SWIZZLE_128B, l2_promotion: int = 2,
                        out: int | None = None) -> TensorMap | None:
    """Encode a 2-D row-major tensor map; into ``out`` (a 64-byte aligned host
    address) if given, else into a fresh TensorMap that is returned."""
    tmap = None
    if out is None:
        tmap = aligned_struct(TensorMap)
        out = C.addressof(tmap)
    call("mtb_tensormap_encode_2d", out, elem_bytes, int(is_float), int(is_bf16),
         base, dim_inner, dim_outer, stride_outer_bytes, box_inner, box_outer, swizzle,
         l2_promotion)
    return tmap


# ------------------------------------------------------------------ streams, events, memory

class Stream:
    def __init__(self) -> None:
        self.handle = C.c_void_p()
        call("mtb_stream_create", C.byref(self.handle))

    @property
    def value(self) -> int:
        return self.handle.value or 0

    def synchronize(self) -> None:
        call("mtb_stream_sync", self.handle)

    def close(self) -> None:
        if self.handle:
            call("mtb_stream_destroy", self.handle)
            self.handle = C.c_void_p()


class Event:
    def __init__(self) -> None:
        self.handle = C.c_void_p()
        call("mtb_event_create", C.byref(self.handle))

    def record(self, stream: int = 0) -> "Event":
        call("mtb_event_record", self.handle, C.c_void_p(stream))
        return self

    def synchronize(self) -> None:
        call("mtb_event_sync", self.handle)

    def elapsed_ms(self, later: "Event") -> float:
        ms = C.c_float()
        call("mtb_event_elapsed_ms", self.handle, later.handle, C.byref(ms))
        return ms.value

    def close(self) -> None:
        if self.handle:
            call("mtb_event_destroy", self.handle)
            self.handle = C.c_void_p()


def mem_alloc(nbytes: int) -> int:
    ptr = C.c_uint64()
    call("mtb_mem_alloc", C.byref(ptr), nbytes)
    return ptr.value


def mem_free(ptr: int) -> None:
    call("mtb_mem_free", C.c_uint64(ptr))


def memcpy_h2d(dst: int, src_address: int, nbytes: int, stream: int = 0) -> None:
    call("mtb_memcpy_h2d", C.c_uint64(dst), C.c_void_p(src_address), nbytes, C.c_void_p(stream))


def memcpy_d2h(dst_address: int, src: int, nbytes: int, stream: int = 0) -> None:
    call("mtb_memcpy_d2h", C.c_void_p(dst_address), C.c_uint64(src), nbytes, C.c_void_p(stream))


def memcpy_d2d(dst: int, src: int, nbytes: int, stream: int = 0) -> None:
    call("mtb_memcpy_d2d", C.c_uint64(dst), C.c_uint64(src), nbytes, C.c_void_p(stream))


def memset_u32(dst: int, value: int, count: int, stream: int = 0) -> None:
    call("mtb_memset_u32", C.c_uint64(dst), C.c_uint32(value), count, C.c_void_p(stream))


def stream_synchronize(stream: int = 0) -> None:
    call("mtb_stream_sync", C.c_void_p(stream))


def status_check(status_ptr: int, stream: int = 0) -> None:
    word = C.c_uint32()
    call("mtb_status_check", C.c_uint64(status_ptr), C.c_void_p(stream), C.byref(word))
