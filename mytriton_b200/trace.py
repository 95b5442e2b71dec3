"""The user-facing kernel language: ``tl.*`` functions, symbolic values, builder.

Calling these functions does not compute anything; it grows an expression tree
(nodes.py) that the SSA lowering consumes.  The surface mirrors the reference's
``src/mytriton/trace.py:13-158`` (functions) and ``:425-515`` (``Value``,
``Ptr``, ``Builder``); ``dot`` and bf16 pointers are additions.
"""

from __future__ import annotations

from typing import TYPE_CHECKING, Annotated, Any, TypeAlias, get_args, get_origin

import numpy as np

from . import arrays
from .nodes import (  # noqa: F401  (re-exported: tests import node classes from here)
    AddPtr, Arange, BinOp, Const, Dot, Empty, ExpandDims, Expression, ForRange, Full,
    Load, LoopCarry, LoopIndex, LoopResult, Max, Maximum, Min, Minimum, Param,
    NumPrograms, ProgramId, Store, Sum, TopLevelOp, UnaryOp, Where, Zeros,
)
from .types import (  # noqa: F401
    BF16, BOOL, F16, F32, I32, PTR_BF16, PTR_F16, PTR_F32, PTR_F8E4M3, PTR_F8E5M2, BlockType, PointerType, ScalarType, Type,
    VectorType, bfloat16, float8e4nv, float8e5, float16, float32, int1, int32,
)

if TYPE_CHECKING:
    constexpr: TypeAlias = Any
else:

    class constexpr:
        """Annotation marking a kernel parameter as a compile-time constant."""


def is_constexpr_annotation(annotation: object) -> bool:
    if annotation is constexpr:
        return True
    if get_origin(annotation) is Annotated:
        return constexpr in get_args(annotation)[1:]
    return False


# ---------------------------------------------------------------- symbolic values


def unwrap(x: Any) -> Any:
    """Strip the ``Value``/``Ptr`` wrapper; Python numbers become ``Const``."""
    if isinstance(x, (Value, Ptr)):
        return x.expr
    if isinstance(x, (int, float)):
        return Const(x)
    return x


class Value:
    """A symbolic scalar or block.  Operators build ``BinOp``/``UnaryOp`` nodes."""

    def __init__(self, expr: Any) -> None:
        self.expr = expr

    def _bin(self, symbol: str, other: Any, swap: bool = False) -> "Value":
        mine, theirs = self.expr, unwrap(other)
        return Value(BinOp(symbol, theirs, mine) if swap else BinOp(symbol, mine, theirs))

    def __add__(self, other): return self._bin("+", other)
    def __radd__(self, other): return self._bin("+", other, swap=True)
    def __sub__(self, other): return self._bin("-", other)
    def __rsub__(self, other): return self._bin("-", other, swap=True)
    def __mul__(self, other): return self._bin("*", other)
    def __rmul__(self, other): return self._bin("*", other, swap=True)
    def __truediv__(self, other): return self._bin("/", other)
    def __rtruediv__(self, other): return self._bin("/", other, swap=True)
    # i32 only, C semantics; spelled as words so that a hand-built BinOp("%", ...) is still the
    # unknown operator the reference's type checker rejects
    def __floordiv__(self, other): return self._bin("floordiv", other)
    def __rfloordiv__(self, other): return self._bin("floordiv", other, swap=True)
    def __mod__(self, other): return self._bin("rem", other)
    def __rmod__(self, other): return self._bin("rem", other, swap=True)
    def __lt__(self, other): return self._bin("<", other)
    def __gt__(self, other): return self._bin("<", other, swap=True)    # a > b is b < a; also serves 3 < a
    def __and__(self, other): return self._bin("&", other)
    def __rand__(self, other): return self._bin("&", other, swap=True)

    def __neg__(self) -> "Value":
        return Value(UnaryOp("neg", self.expr))

    def __invert__(self) -> "Value":
        return Value(UnaryOp("not", self.expr))     # booleans only (checked by type inference)

    def to(self, dtype: Any) -> "Value":
        """``x.to(tl.float32)``: integers become floats, floats stay.  ``x.to(tl.float16)`` /
        ``x.to(tl.bfloat16)``: the value rounded to that precision (nearest even) — registers hold
        fp32 throughout, so this is what a later store to a 16-bit array would do anyway."""
        from .type_inference import TypeInference
        from .types import BF16, F16, F32, I32, element_of

        element = element_of(TypeInference().infer(self.expr))
        if dtype == I32:
            if element == I32:
                return self
            raise TypeError("conversion of floating-point values to int32 is not supported")
        if dtype not in (F32, F16, BF16):
            raise TypeError(f"unsupported conversion target: {dtype}")
        if element not in (F32, I32):
            raise TypeError(f"cannot convert {element} values")
        as_float = self if element == F32 else self * 1.0
        if dtype == F32:
            return as_float
        return Value(UnaryOp("round_f16" if dtype == F16 else "round_bf16", as_float.expr))

    def __bool__(self) -> bool:
        raise TypeError(
            "Python control flow over symbolic values is not supported; "
            "when combining comparisons with &, wrap each comparison in parentheses"
        )

    def __getitem__(self, index) -> "Value":
        if isinstance(index, tuple) and len(index) == 2:
            first, second = index
            if first == slice(None) and second is None:
                return Value(ExpandDims(self.expr, axis=1))
            if first is None and second == slice(None):
                return Value(ExpandDims(self.expr, axis=0))
        raise TypeError("only x[:, None] and x[None, :] are supported for symbolic values")

    def __repr__(self) -> str:
        return f"Value({self.expr})"


class Ptr:
    """A symbolic pointer (scalar or block of pointers); only ``+ offset`` exists."""

    def __init__(self, expr: Any) -> None:
        self.expr = expr

    def __add__(self, offset) -> "Ptr":
        return Ptr(AddPtr(self.expr, unwrap(offset)))

    def __repr__(self) -> str:
        return f"Ptr({self.expr})"


class Builder:
    """Collects the side-effecting top-level ops (stores, loops) while tracing."""

    _current: "Builder | None" = None

    def __init__(self) -> None:
        self.ops: list[Any] = []
        self._previous: "Builder | None" = None

    def __enter__(self) -> "Builder":
        self._previous, Builder._current = Builder._current, self
        return self

    def __exit__(self, exc_type, exc, tb) -> None:
        Builder._current = self._previous

    @staticmethod
    def current() -> "Builder":
        assert Builder._current is not None
        return Builder._current


# ---------------------------------------------------------------- runtime-if predication
#
# ``if`` on a run-time scalar is lowered by predication: both branches are traced, every
# load and store traced inside a branch gets the branch condition ANDed into its mask, and
# names assigned in a branch are merged with ``where``.  ``return`` under a condition adds
# a filter that every later memory operation carries.  The IR needs no branch construct.


class _Guards:
    def __init__(self) -> None:
        self.stack: list[Any] = []      # conjunction in force inside the innermost branch
        self.exits: list[Any] = []      # negated conditions of the returns traced so far
        self.current: Any | None = None

    def refresh(self) -> None:
        terms = self.stack[-1:] + self.exits
        self.current = None
        for term in terms:
            self.current = term if self.current is None else BinOp("&", self.current, term)


_guards = _Guards()


class guards_reset:
    """Fresh predication state for one kernel trace."""

    def __enter__(self) -> None:
        _guards.__init__()

    def __exit__(self, exc_type, exc, tb) -> None:
        _guards.__init__()


class predicated:
    """While active, memory operations are masked by ``condition`` (an expression that
    already includes the enclosing branches' conditions)."""

    def __init__(self, condition: Any) -> None:
        self.condition = condition

    def __enter__(self) -> None:
        _guards.stack.append(self.condition)
        _guards.refresh()

    def __exit__(self, exc_type, exc, tb) -> None:
        _guards.stack.pop()
        _guards.refresh()


def branch_predicate() -> Any | None:
    """Condition of the innermost active branch (None outside any run-time ``if``)."""
    return _guards.stack[-1] if _guards.stack else None


def active_predicate() -> Any | None:
    """Everything a memory operation traced now must be masked by."""
    return _guards.current


def add_exit(condition_not_taken: Any) -> None:
    _guards.exits.append(condition_not_taken)
    _guards.refresh()


def _guard(mask: Any) -> Any:
    predicate = _guards.current
    if predicate is None:
        return mask
    return predicate if mask is None else BinOp("&", mask, predicate)


# ---------------------------------------------------------------- language functions


def program_id(axis: int) -> Value:
    return Value(ProgramId(axis))


def trans(value: Value) -> Value:
    """The transpose of a rank-2 block (``tl.dot(q, tl.trans(k))``).  It costs nothing by itself:
    whatever produces the block is instantiated with its two coordinates exchanged."""
    return Value(UnaryOp("trans", unwrap(value)))


def num_programs(axis: int) -> Value:
    """The launch grid's extent along ``axis``: with ``program_id`` it lets a kernel stride over
    more work items than it has programs."""
    return Value(NumPrograms(axis))


def arange(start: int, end: int) -> Value:
    return Value(Arange(start, end))


def _block_shape(shape) -> tuple[int, ...]:
    if type(shape) is int:
        shape = (shape,)
    elif isinstance(shape, list):
        shape = tuple(shape)
    if not isinstance(shape, tuple) or len(shape) == 0:
        raise TypeError(f"block shape must be a non-empty int sequence, got {shape!r}")
    for dim in shape:
        if type(dim) is not int or dim <= 0:
            raise TypeError(f"block dimensions must be positive integers, got {shape}")
    return shape


def _block_dtype(dtype: ScalarType) -> ScalarType:
    if dtype not in (BOOL, I32, F32):
        raise TypeError(f"block dtype must be int1, int32, or float32, got {dtype}")
    return dtype


def empty(shape: "int | tuple[int, ...] | list[int]", dtype: ScalarType) -> Value:
    return Value(Empty(_block_shape(shape), _block_dtype(dtype)))


def zeros(shape: "int | tuple[int, ...] | list[int]", dtype: ScalarType) -> Value:
    return Value(Zeros(_block_shape(shape), _block_dtype(dtype)))


def full(shape: "int | tuple[int, ...] | list[int]", value: "Value | bool | int | float",
         dtype: ScalarType) -> Value:
    return Value(Full(_block_shape(shape), unwrap(value), _block_dtype(dtype)))


def _opt(x: Any) -> Any:
    return None if x is None else unwrap(x)


def load(ptr: "Ptr", mask: "Value | bool | None" = None,
         other: "Value | int | float | None" = None) -> Value:
    return Value(Load(ptr=unwrap(ptr), mask=_guard(_opt(mask)), other=_opt(other)))


def store(ptr: "Ptr", value: "Value | int | float", mask: "Value | bool | None" = None) -> None:
    Builder.current().ops.append(Store(ptr=unwrap(ptr), value=unwrap(value), mask=_guard(_opt(mask))))


def atomic_add(ptr: "Ptr", value: "Value | int | float", mask: "Value | bool | None" = None) -> None:
    """Add ``value`` to the f32 or i32 elements ``ptr`` points at, atomically with respect to
    every other program (the old values are not returned).  Floating-point sums then depend
    on the order in which programs arrive."""
    Builder.current().ops.append(
        Store(ptr=unwrap(ptr), value=unwrap(value), mask=_guard(_opt(mask)), atomic=True))


def maximum(lhs: "Value | int | float", rhs: "Value | int | float") -> Value:
    return Value(Maximum(unwrap(lhs), unwrap(rhs)))


def minimum(lhs: "Value | int | float", rhs: "Value | int | float") -> Value:
    return Value(Minimum(unwrap(lhs), unwrap(rhs)))


def exp(value: "Value | float") -> Value:
    return Value(UnaryOp("exp", unwrap(value)))


def _float_unary(name: str):
    def function(value: "Value | float") -> Value:
        return Value(UnaryOp(name, unwrap(value)))

    function.__name__ = function.__qualname__ = name
    function.__doc__ = f"Elementwise ``{name}`` of an f32 scalar or block."
    return function


sqrt, rsqrt, log, log2, exp2, sin, cos, tanh = (
    _float_unary(name) for name in ("sqrt", "rsqrt", "log", "log2", "exp2", "sin", "cos", "tanh"))


def abs(value: "Value | int | float") -> Value:      # noqa: A001 - the language's name
    """Elementwise absolute value: ``fabsf`` on f32, a select on i32."""
    return Value(UnaryOp("abs", unwrap(value)))


def sigmoid(value: "Value | float") -> Value:
    """``1 / (1 + exp(-x))``, composed from the primitive ops."""
    return 1.0 / (1.0 + exp(-Value(unwrap(value))))


def cdiv(x, y):
    """Ceiling division of non-negative ints: a Python int for compile-time operands."""
    return (x + y - 1) // y


def where(condition: "Value | bool", true_value: "Value | int | float",
          false_value: "Value | int | float") -> Value:
    return Value(Where(unwrap(condition), unwrap(true_value), unwrap(false_value)))


def sum(value: Value, axis: int | None = None) -> Value:  # noqa: A001 - name fixed by the language
    """Sum of a rank-1 block (a scalar), or of a rank-2 block along ``axis`` (a rank-1 block)."""
    return Value(Sum(unwrap(value), axis))


def max(value: Value, axis: int | None = None) -> Value:  # noqa: A001
    return Value(Max(unwrap(value), axis))


def min(value: Value, axis: int | None = None) -> Value:  # noqa: A001
    return Value(Min(unwrap(value), axis))


def dot(a: Value, b: Value, acc: Value | None = None, input_precision: str | None = None) -> Value:
    """Tile product ``a[BM,BK] @ b[BK,BN]`` accumulated in fp32 (plus ``acc``).

    ``input_precision="tf32"`` lets fp32 operands go through the tensor cores with their
    mantissas cut to 10 bits; the default ("ieee") keeps fp32 operands exact."""
    precision = "ieee" if input_precision is None else input_precision
    if precision not in ("ieee", "tf32"):
        raise ValueError(f"input_precision must be 'ieee' or 'tf32', got {input_precision!r}")
    return Value(Dot(unwrap(a), unwrap(b), _opt(acc), precision))


def static_range(start: int, stop: int | None = None, step: int = 1) -> range:
    if stop is None:
        start, stop = 0, start
    for label, bound in zip(("start", "stop", "step"), (start, stop, step)):
        if not isinstance(bound, int):
            raise ValueError(
                f"static_range {label} must be compile-time int, got {type(bound).__name__}"
            )
    return range(start, stop, step)


# ---------------------------------------------------------------- runtime parameters

_POINTER_FOR_DTYPE = {"float32": PTR_F32, "bfloat16": PTR_BF16, "float16": PTR_F16,
                      "float8_e4m3fn": PTR_F8E4M3, "float8_e5m2": PTR_F8E5M2}


_UNSET = object()


def _make_param(name: str, value: Any, info: Any = _UNSET) -> Param:
    if info is _UNSET:
        info = arrays.describe(value)
    if info is not None:
        pointer = _POINTER_FOR_DTYPE.get(info.dtype)
        if pointer is None:
            raise TypeError(f"{name}: only float32 arrays are supported")
        if not info.contiguous:
            raise TypeError(f"{name}: only C-contiguous arrays are supported")
        return Param(name, pointer)
    if isinstance(value, (int, np.integer)):
        return Param(name, I32)
    if isinstance(value, (float, np.floating)):
        return Param(name, F32)
    raise TypeError(f"{name}: unsupported runtime value {type(value)}")


def make_runtime_params(signature, bound_args) -> list[Param]:
    return [
        _make_param(name, bound_args[name])
        for name, parameter in signature.parameters.items()
        if not is_constexpr_annotation(parameter.annotation)
    ]

