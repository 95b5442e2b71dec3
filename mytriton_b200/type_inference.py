"""Static types of expression-tree nodes.

Rules follow the reference's ``src/mytriton/type_inference.py:92-275``: numeric
promotion (f32 wins over i32), NumPy-style shape broadcast, bool-only masks,
i32-only pointer offsets, rank-1-only reductions.  Additions: bf16 promotes to
f32 in arithmetic, and ``Dot`` takes ``[BM,BK] x [BK,BN] -> [BM,BN] f32``.
Results are memoised by node identity in ``self.types`` (the SSA lowering
snapshots and restores that dict around loops).
"""

from __future__ import annotations

from . import nodes as N
from .block_shapes import broadcast_shapes
from .types import (
    BF16, BOOL, BYTE_WIDTH, F16, F32, FLOAT_UNARY, I32, NUMERIC, BlockType, PointerType, ScalarType, Type, element_of,
)


class TypeInference:
    ARITHMETIC_OPS = {"+", "-", "*", "/"}

    def __init__(self) -> None:
        self.types: dict[int, Type] = {}

    # -- helpers -----------------------------------------------------------------

    def element_type(self, ty: Type):
        return element_of(ty)

    def with_shape(self, element, *types: Type) -> Type:
        shapes = [ty.shape for ty in types if isinstance(ty, BlockType)]
        if not shapes:
            return element
        try:
            return BlockType(broadcast_shapes(*shapes), element)
        except ValueError as error:
            raise TypeError(f"Cannot broadcast shapes: {shapes}") from error

    def promote(self, lhs: Type, rhs: Type) -> ScalarType:
        pair = (element_of(lhs), element_of(rhs))
        if pair[0] not in NUMERIC or pair[1] not in NUMERIC:
            raise TypeError(f"Cannot combine {lhs} and {rhs}")
        return I32 if pair == (I32, I32) else F32

    def require_mask(self, mask: Type) -> None:
        if element_of(mask) != BOOL:
            raise TypeError(f"Mask must be bool, got {mask}")

    def require_convertible(self, source: Type, destination: ScalarType, *, context: str) -> None:
        have = element_of(source)
        if have == destination or (have in NUMERIC and destination in NUMERIC):
            return
        raise TypeError(f"{context} must be convertible to {destination}, got {source}")

    # -- entry point -------------------------------------------------------------

    def infer(self, expr) -> Type:
        key = id(expr)
        known = self.types.get(key)
        if known is not None:
            return known
        rule = getattr(self, "_ty_" + type(expr).__name__, None)
        if rule is None:
            raise TypeError(f"Cannot infer type of {expr}")
        ty = rule(expr)
        self.types[key] = ty
        return ty

    # -- leaves ------------------------------------------------------------------

    def _ty_Const(self, e: N.Const) -> Type:
        for python_type, ty in ((bool, BOOL), (int, I32), (float, F32)):
            if isinstance(e.value, python_type):
                return ty
        raise TypeError(f"Unsupported constant: {e.value!r}")

    def _ty_Param(self, e: N.Param) -> Type:
        return e.ty

    def _ty_ProgramId(self, e) -> Type:
        return I32

    def _ty_NumPrograms(self, e) -> Type:
        return I32

    def _ty_LoopIndex(self, e) -> Type:
        return I32

    def _ty_LoopCarry(self, e: N.LoopCarry) -> Type:
        return self.infer(e.initial)

    def _ty_LoopResult(self, e: N.LoopResult) -> Type:
        return self.infer(e.loop.carried_outputs[e.index])

    def _ty_Arange(self, e: N.Arange) -> Type:
        if e.end <= e.start:
            raise TypeError(f"arange requires end > start, got [{e.start}, {e.end})")
        return BlockType((e.end - e.start,), I32)

    def _ty_Empty(self, e) -> Type:
        return BlockType(e.shape, e.dtype)

    _ty_Zeros = _ty_Empty

    def _ty_Full(self, e: N.Full) -> Type:
        fill = self.infer(e.value)
        if isinstance(fill, BlockType):
            raise TypeError(f"full value must be scalar, got {fill}")
        self.require_convertible(fill, e.dtype, context="full value")
        return BlockType(e.shape, e.dtype)

    # -- operators ---------------------------------------------------------------

    def _ty_BinOp(self, e: N.BinOp) -> Type:
        lhs, rhs = self.infer(e.lhs), self.infer(e.rhs)
        if e.op == "<":
            self.promote(lhs, rhs)
            return self.with_shape(BOOL, lhs, rhs)
        if e.op == "&":
            if element_of(lhs) != BOOL or element_of(rhs) != BOOL:
                raise TypeError(f"& expects bool operands, got {lhs} and {rhs}")
            return self.with_shape(BOOL, lhs, rhs)
        if e.op in self.ARITHMETIC_OPS:
            return self.with_shape(self.promote(lhs, rhs), lhs, rhs)
        if e.op in ("floordiv", "rem"):
            if element_of(lhs) != I32 or element_of(rhs) != I32:
                raise TypeError(f"{e.op} expects i32 operands, got {lhs} and {rhs}")
            return self.with_shape(I32, lhs, rhs)
        raise TypeError(f"Unsupported binary operator: {e.op!r}")

    def _ty_Maximum(self, e) -> Type:
        lhs, rhs = self.infer(e.lhs), self.infer(e.rhs)
        return self.with_shape(self.promote(lhs, rhs), lhs, rhs)

    _ty_Minimum = _ty_Maximum

    def _ty_UnaryOp(self, e: N.UnaryOp) -> Type:
        operand = self.infer(e.value)
        element = element_of(operand)
        if e.op == "neg":
            if element not in NUMERIC:
                raise TypeError(f"Cannot negate {operand}")
        elif e.op == "exp":
            if element != F32:
                raise TypeError(f"exp requires f32, got {operand}")
        elif e.op == "abs":
            if element not in NUMERIC:
                raise TypeError(f"Cannot take abs of {operand}")
        elif e.op in FLOAT_UNARY:
            if element != F32:
                raise TypeError(f"{e.op} requires f32, got {operand}")
        elif e.op == "not":
            if element != BOOL:
                raise TypeError(f"not requires a boolean, got {operand}")
        elif e.op == "trans":
            if not isinstance(operand, BlockType) or operand.rank != 2:
                raise TypeError(f"trans expects a rank-2 block, got {operand}")
            return BlockType((operand.shape[1], operand.shape[0]), operand.element)
        else:
            raise TypeError(f"Unknown unary operation: {e.op}")
        return operand

    def _ty_Where(self, e: N.Where) -> Type:
        condition = self.infer(e.condition)
        if element_of(condition) != BOOL:
            raise TypeError(f"where condition must be bool, got {condition}")
        yes, no = self.infer(e.true_value), self.infer(e.false_value)
        return self.with_shape(self.promote(yes, no), condition, yes, no)

    def _reduction(self, e) -> Type:
        operand = self.infer(e.value)
        axis = getattr(e, "axis", None)
        if isinstance(operand, BlockType) and operand.rank == 2 and axis is not None:
            if axis not in (0, 1):
                raise TypeError(f"invalid reduction axis {axis} for {operand}")
            if operand.element not in (I32, F32):
                raise TypeError(f"cannot reduce elements of type {operand.element}")
            return BlockType((operand.shape[1 - axis],), operand.element)
        if not isinstance(operand, BlockType) or operand.rank != 1 or axis not in (None, 0):
            raise TypeError(f"{type(e).__name__} expects vector, got {operand}")
        if operand.element not in (I32, F32):
            raise TypeError(f"cannot reduce elements of type {operand.element}")
        return operand.element

    _ty_Sum = _ty_Max = _ty_Min = _reduction

    def _ty_ExpandDims(self, e: N.ExpandDims) -> Type:
        operand = self.infer(e.value)
        if not isinstance(operand, BlockType):
            raise TypeError(f"expand_dims expects block, got {operand}")
        if not 0 <= e.axis <= operand.rank:
            raise TypeError(f"invalid expand_dims axis {e.axis} for {operand}")
        dims = list(operand.shape)
        dims.insert(e.axis, 1)
        return BlockType(tuple(dims), operand.element)

    def _ty_Dot(self, e: N.Dot) -> Type:
        lhs, rhs = self.infer(e.lhs), self.infer(e.rhs)
        for side, ty in (("lhs", lhs), ("rhs", rhs)):
            if not isinstance(ty, BlockType) or ty.rank != 2 or ty.element not in (F32, BF16, F16) + BYTE_WIDTH:
                raise TypeError(f"dot {side} must be a rank-2 f32/bf16/f16/fp8 block, got {ty}")
        if lhs.element != rhs.element:
            raise TypeError(f"dot operands must share one element type, got {lhs} and {rhs}")
        if lhs.shape[1] != rhs.shape[0]:
            raise TypeError(f"dot inner dimensions differ: {lhs} and {rhs}")
        result = BlockType((lhs.shape[0], rhs.shape[1]), F32)
        if e.acc is not None:
            acc = self.infer(e.acc)
            if acc != result:
                raise TypeError(f"dot accumulator must be {result}, got {acc}")
        return result

    # -- memory ------------------------------------------------------------------

    def _ty_AddPtr(self, e: N.AddPtr) -> Type:
        base, offset = self.infer(e.base), self.infer(e.offset)
        pointer = element_of(base)
        if not isinstance(pointer, PointerType):
            raise TypeError(f"Expected pointer, got {base}")
        if element_of(offset) != I32:
            raise TypeError(f"Pointer offset must be i32, got {offset}")
        return self.with_shape(pointer, base, offset)

    def _ty_Load(self, e: N.Load) -> Type:
        ptr = self.infer(e.ptr)
        pointer = element_of(ptr)
        if not isinstance(pointer, PointerType):
            raise TypeError(f"Cannot load from {ptr}")
        shaped = [ptr]
        if e.mask is not None:
            mask = self.infer(e.mask)
            self.require_mask(mask)
            shaped.append(mask)
        if e.other is not None:
            other = self.infer(e.other)
            self.require_convertible(other, pointer.element, context="Load fallback")
            shaped.append(other)
        return self.with_shape(pointer.element, *shaped)

    def check_break_unless(self, op: N.BreakUnless) -> None:
        condition = self.infer(op.condition)
        if condition != BOOL:
            raise TypeError(f"a loop condition must be a scalar boolean, got {condition}")

    def check_store(self, store: N.Store) -> None:
        ptr, value = self.infer(store.ptr), self.infer(store.value)
        pointer = element_of(ptr)
        if not isinstance(pointer, PointerType):
            raise TypeError(f"Cannot store to {ptr}")
        self.require_convertible(value, pointer.element, context="Stored value")
        if store.atomic and pointer.element not in (F32, I32):
            raise TypeError(f"atomic_add needs an f32 or i32 array, got {ptr}")
        shaped = [ptr, value]
        if store.mask is not None:
            mask = self.infer(store.mask)
            self.require_mask(mask)
            shaped.append(mask)
        self.with_shape(pointer.element, *shaped)
