"""Uniform view of the array objects a kernel may be called with.

NumPy arrays (host, compile-only), ``torch`` tensors, and anything exposing
``__cuda_array_interface__`` are accepted; nothing here imports torch or any
GPU library, objects are recognised by duck typing.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any


@dataclass(frozen=True)
class ArrayInfo:
    dtype: str          # "float32", "bfloat16", ...
    contiguous: bool
    on_device: bool
    address: int | None  # device or host address; None if unknown


_dtype_names: dict[Any, str] = {}


def _dtype_name(dtype: Any) -> str:
    """``str(dtype)`` without the ``torch.`` prefix, memoised (NumPy's is slow)."""
    try:
        return _dtype_names[dtype]
    except (KeyError, TypeError):
        text = str(dtype)
        if text.startswith("torch."):
            text = text.split(".", 1)[1]
        try:
            _dtype_names[dtype] = text
        except TypeError:
            pass
        return text


def describe(value: Any) -> ArrayInfo | None:
    """Return an ArrayInfo for array-like ``value`` or None for scalars."""
    module = type(value).__module__
    if module.startswith("torch") and hasattr(value, "data_ptr"):
        return ArrayInfo(
            dtype=_dtype_name(value.dtype),
            contiguous=bool(value.is_contiguous()),
            on_device=bool(value.is_cuda),
            address=int(value.data_ptr()) if value.numel() else 0,
        )
    cai = getattr(value, "__cuda_array_interface__", None)
    if cai is not None:
        strides = cai.get("strides")
        contiguous = strides is None or bool(getattr(value, "c_contiguous", False))
        dtype = getattr(value, "dtype_name", None) or _typestr_name(cai["typestr"])
        return ArrayInfo(dtype, contiguous, True, int(cai["data"][0] or 0))
    if hasattr(value, "dtype") and hasattr(value, "flags"):
        address = None
        iface = getattr(value, "__array_interface__", None)
        if iface is not None:
            address = int(iface["data"][0])
        return ArrayInfo(
            dtype=_dtype_name(value.dtype),
            contiguous=bool(value.flags.c_contiguous),
            on_device=_is_foreign_device_array(value),
            address=address,
        )
    return None


def _is_foreign_device_array(value: Any) -> bool:
    module = type(value).__module__
    return module == "cupy" or module.startswith("cupy.")


def _typestr_name(typestr: str) -> str:
    return {"<f4": "float32", "<i4": "int32", "<f2": "float16", "<u2": "bfloat16"}.get(
        typestr, typestr
    )


def element_count(value: Any) -> int:
    """Number of elements of an array argument (torch tensor, DeviceArray, NumPy array or
    anything that publishes ``__cuda_array_interface__``)."""
    numel = getattr(value, "numel", None)
    if callable(numel):
        return int(numel())
    size = getattr(value, "size", None)
    if isinstance(size, int):
        return size
    iface = getattr(value, "__cuda_array_interface__", None)
    if iface is not None:
        count = 1
        for extent in iface["shape"]:
            count *= int(extent)
        return count
    raise TypeError(f"cannot tell the size of {type(value).__name__}")
