"""Shape arithmetic shared by type inference, the verifier and the code generator.

``broadcast_shapes`` keeps the reference's NumPy-style rule and error text
(``src/mytriton/block_shapes.py:18-36``).  ``cuda_kernel_block_shape`` and
``cuda_threads_per_block`` reproduce the reference's *legacy* launch geometry
(``:55-114``: one thread per logical element, at most 1024) — this backend does
not launch that way, but the functions remain for code that asks what the
reference would have done (for instance when launching reference-generated
source), and ``cuda_kernel_block_shape`` still supplies the "one vector width
per rank-1 kernel" diagnostic.
"""

from __future__ import annotations

from itertools import zip_longest
from math import prod as _prod

from .types import BlockType


def prod(shape: tuple[int, ...]) -> int:
    return _prod(shape)


def _render(shape: tuple[int, ...]) -> str:
    return "x".join(str(dim) for dim in shape)


def broadcast_shapes(*shapes: tuple[int, ...]) -> tuple[int, ...]:
    """Right-aligned broadcast; every dimension may hold at most one non-1 extent."""
    out: list[int] = []
    for extents in zip_longest(*(reversed(shape) for shape in shapes), fillvalue=1):
        distinct = {extent for extent in extents if extent != 1}
        if len(distinct) > 1:
            raise ValueError(
                "cannot broadcast shapes: " + ", ".join(_render(shape) for shape in shapes)
            )
        out.append(distinct.pop() if distinct else 1)
    return tuple(reversed(out))


def result_block_shapes(ssa_ops) -> list[tuple[int, ...]]:
    """Shapes of every block-typed SSA result, loop bodies included, in order."""
    found: list[tuple[int, ...]] = []
    for item in ssa_ops:
        body = getattr(item, "body", None)
        if body is not None:
            found += result_block_shapes(body)
        elif item.result is not None and isinstance(item.result.ty, BlockType):
            found.append(item.result.ty.shape)
    return found


def cuda_kernel_block_shape(ssa_ops) -> tuple[int, ...]:
    shapes = result_block_shapes(ssa_ops)
    if not shapes:
        return (1,)
    if max(len(shape) for shape in shapes) > 2:
        raise ValueError(
            "CUDA lowering supports only rank-1/rank-2 blocks, got "
            + ", ".join(str(shape) for shape in shapes)
        )
    tiles = [shape for shape in shapes if len(shape) == 2]
    widths = [shape[0] for shape in shapes if len(shape) == 1]
    if not tiles:
        if len(set(widths)) != 1:
            raise ValueError(
                "CUDA lowering requires one vector width, got: "
                + ", ".join(str(width) for width in sorted(set(widths)))
            )
        return (widths[0],)
    tile = broadcast_shapes(*tiles)
    legal = {tile[0], tile[1], tile[0] * tile[1]}
    stray = [width for width in widths if width not in legal]
    if stray:
        raise ValueError(
            "rank-1 block widths in a rank-2 CUDA kernel must match one tile "
            f"dimension or full tile size; got {stray}, tile shape is {tile}"
        )
    return tile


def cuda_threads_per_block(ssa_ops) -> int:
    threads = prod(cuda_kernel_block_shape(ssa_ops))
    if not 1 <= threads <= 1024:
        raise ValueError(
            f"CUDA threads per block must be between 1 and 1024, got {threads}"
        )
    return threads
