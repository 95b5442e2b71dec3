"""Type rules of the expression tree (CPU).  The rules are the reference's
(src/mytriton/type_inference.py:92-275); bf16/f16 and Dot are additions."""

import pytest

import mytriton_b200.language as tl
from mytriton_b200.nodes import AddPtr, Arange, BinOp, Const, Dot, ExpandDims, Full, Load, Param, Store
from mytriton_b200.trace import Value
from mytriton_b200.type_inference import TypeInference
from mytriton_b200.types import (
    BF16, BOOL, F16, F32, I32, PTR_BF16, PTR_F32, BlockType, PointerType, VectorType,
)

X = Param("x", PTR_F32)


def infer(expr):
    return TypeInference().infer(expr)


def test_constants_and_scalars():
    assert infer(Const(True)) == BOOL and infer(Const(3)) == I32 and infer(Const(1.5)) == F32
    with pytest.raises(TypeError, match="Unsupported constant"):
        infer(Const("text"))
    assert infer(Param("n", I32)) == I32 and infer(tl.program_id(0).expr) == I32


def test_promotion_and_broadcast():
    lanes = Arange(0, 8)
    assert infer(BinOp("+", lanes, Const(1))) == VectorType(8, I32)
    assert infer(BinOp("*", lanes, Const(0.5))) == VectorType(8, F32)
    assert infer(BinOp("/", Const(7), Const(2))) == I32               # i32 / i32 stays i32
    rows, cols = ExpandDims(Arange(0, 4), 1), ExpandDims(Arange(0, 8), 0)
    assert infer(BinOp("+", rows, cols)) == BlockType((4, 8), I32)
    assert infer(BinOp("+", rows, Arange(0, 8))) == BlockType((4, 8), I32)   # rank-1 pads on the left
    with pytest.raises(TypeError, match="Cannot broadcast"):
        infer(BinOp("+", Arange(0, 4), Arange(0, 8)))
    with pytest.raises(TypeError, match="Cannot combine bool and bool"):
        infer(BinOp("+", Const(True), Const(False)))
    with pytest.raises(TypeError, match="Unsupported binary operator"):
        infer(BinOp("%", Const(1), Const(2)))


def test_comparisons_and_masks():
    lanes = Arange(0, 8)
    less = BinOp("<", lanes, Param("n", I32))
    assert infer(less) == VectorType(8, BOOL)
    assert infer(BinOp("&", less, less)) == VectorType(8, BOOL)
    with pytest.raises(TypeError, match="& expects bool operands"):
        infer(BinOp("&", lanes, less))


def test_pointers_loads_and_stores():
    ptr = AddPtr(X, Arange(0, 8))
    assert infer(ptr) == VectorType(8, PTR_F32)
    assert infer(Load(ptr, None, None)) == VectorType(8, F32)
    assert infer(Load(X, BinOp("<", Arange(0, 4), Const(2)), Const(0.0))) == VectorType(4, F32)
    with pytest.raises(TypeError, match="Expected pointer"):
        infer(AddPtr(Param("n", I32), Const(1)))
    with pytest.raises(TypeError, match="Pointer offset must be i32"):
        infer(AddPtr(X, Const(1.0)))
    with pytest.raises(TypeError, match="Cannot load from f32"):
        infer(Load(Param("v", F32), None, None))
    with pytest.raises(TypeError, match="Mask must be bool"):
        infer(Load(ptr, Arange(0, 8), None))
    with pytest.raises(TypeError, match="Load fallback must be convertible to f32"):
        infer(Load(ptr, None, Const(True)))
    # (types are memoised by node identity, so each tree gets its own checker)
    def check(store):
        TypeInference().check_store(store)

    check(Store(ptr, Arange(0, 8), None))                             # i32 value into f32 memory
    check(Store(Param("flag", PointerType(BOOL)), Const(True), None))
    with pytest.raises(TypeError, match="Stored value must be convertible to bool"):
        check(Store(Param("flag", PointerType(BOOL)), Const(1), None))
    with pytest.raises(TypeError, match="Cannot store to i32"):
        check(Store(Param("n", I32), Const(1), None))
    with pytest.raises(TypeError, match="Cannot broadcast"):
        check(Store(ptr, Arange(0, 4), None))


def test_unary_where_and_extrema():
    value = Value(Param("v", F32))
    assert infer(tl.exp(value).expr) == F32 and infer((-value).expr) == F32
    with pytest.raises(TypeError, match="exp requires f32, got i32"):
        infer(tl.exp(Value(Param("n", I32))).expr)
    with pytest.raises(TypeError, match="Cannot negate bool"):
        infer((-Value(Const(True))).expr)
    lanes = Value(Arange(0, 4))
    assert infer(tl.where(lanes < 2, lanes, 0.5).expr) == VectorType(4, F32)
    with pytest.raises(TypeError, match="where condition must be bool"):
        infer(tl.where(lanes, 1, 2).expr)
    assert infer(tl.maximum(Value(Param("n", I32)), 2.0).expr) == F32
    assert infer(tl.minimum(lanes, 3).expr) == VectorType(4, I32)


def test_reductions_constructors_and_expand_dims():
    lanes = Value(Arange(0, 8))
    assert infer(tl.sum(lanes).expr) == I32 and infer(tl.max(lanes * 1.0).expr) == F32
    with pytest.raises(TypeError, match="expects vector"):
        infer(tl.sum(Value(Param("v", F32))).expr)
    with pytest.raises(TypeError, match="expects vector"):
        infer(tl.min(lanes[:, None]).expr)
    with pytest.raises(TypeError, match="cannot reduce elements of type bool"):
        infer(tl.sum(lanes < 2).expr)
    assert infer(tl.zeros((2, 4), tl.float32).expr) == BlockType((2, 4), F32)
    assert infer(tl.full([8], 3, tl.float32).expr) == VectorType(8, F32)
    with pytest.raises(TypeError, match="full value must be scalar"):
        infer(Full((8,), Arange(0, 8), F32))
    with pytest.raises(TypeError, match=r"block shape|block dimensions"):
        tl.zeros((0,), tl.float32)
    with pytest.raises(TypeError, match="block dtype"):
        tl.zeros((4,), PTR_F32)
    with pytest.raises(TypeError, match="arange requires end > start"):
        infer(Arange(4, 4))
    assert infer(lanes[None, :].expr) == BlockType((1, 8), I32)
    with pytest.raises(TypeError, match="only x"):
        lanes[0]


def test_half_width_types_and_dot():
    a = Load(AddPtr(Param("a", PTR_BF16), BinOp("+", ExpandDims(Arange(0, 16), 1), ExpandDims(Arange(0, 32), 0))), None, None)
    b = Load(AddPtr(Param("b", PTR_BF16), BinOp("+", ExpandDims(Arange(0, 32), 1), ExpandDims(Arange(0, 8), 0))), None, None)
    assert infer(a) == BlockType((16, 32), BF16)
    assert infer(Dot(a, b, None)) == BlockType((16, 8), F32)
    assert infer(BinOp("+", a, Const(1.0))) == BlockType((16, 32), F32)      # arithmetic widens
    with pytest.raises(TypeError, match="dot inner dimensions differ"):
        infer(Dot(a, a, None))
    with pytest.raises(TypeError, match="dot accumulator must be"):
        infer(Dot(a, b, a))
    f16 = Load(AddPtr(Param("h", PointerType(F16)), BinOp("+", ExpandDims(Arange(0, 32), 1), ExpandDims(Arange(0, 8), 0))), None, None)
    with pytest.raises(TypeError, match="share one element type"):
        infer(Dot(a, f16, None))
    with pytest.raises(TypeError, match="rank-2"):
        infer(Dot(Arange(0, 4), b, None))
