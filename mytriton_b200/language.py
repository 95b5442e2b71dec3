"""``import mytriton_b200.language as tl`` — the kernel-language namespace.

Same names as the reference's ``src/mytriton/language.py:1-43`` plus ``dot``
``bfloat16``, ``float16``, ``float8e4nv``, ``float8e5`` and ``num_programs``.
"""

from .trace import (  # noqa: A004 - ``abs``, ``max``, ``min``, ``sum`` are the language's names
    abs, atomic_add, cdiv, cos, exp2, log, log2, rsqrt, sigmoid, sin, sqrt, tanh,
    arange, bfloat16, constexpr, dot, empty, exp, float8e4nv, float8e5, float16, float32, full, int1, int32, load, max,
    maximum, min, minimum, num_programs, program_id, static_range, store, sum, trans, where, zeros,
)

__all__ = [
    "abs", "atomic_add", "cdiv", "cos", "exp2", "log", "log2", "rsqrt", "sigmoid", "sin", "sqrt", "tanh",
    "arange", "bfloat16", "constexpr", "dot", "empty", "exp", "float8e4nv", "float8e5", "float16", "float32", "full", "int1",
    "int32", "load", "max", "maximum", "min", "minimum", "num_programs", "program_id", "static_range",
    "store", "sum", "trans", "where", "zeros",
]
