"""The SSA verifier on hand-built op lists (CPU): arity, results, definition order,
per-opcode typing and the loop-region contract.  Diagnostics keep the reference's
form (src/mytriton/ssa_verification.py:52-53)."""

import pytest

from mytriton_b200.nodes import Const, Param
from mytriton_b200.ssa import SSAForRange, SSAOp, SSAValue
from mytriton_b200.ssa_verification import CompileError, SSAVerifier
from mytriton_b200.types import BF16, BOOL, F32, I32, PTR_F32, BlockType, VectorType

OUT = Param("out", PTR_F32)


def v(i, ty):
    return SSAValue(i, ty)


def verify(ops, block_size=None):
    return SSAVerifier(block_size).verify(ops)


def fails(ops, message, block_size=None):
    with pytest.raises(CompileError, match=message):
        verify(ops, block_size)


def test_structure():
    fails([SSAOp("add", (Const(1), Const(2)), None)], "ssa-verifier: op #0 'add': missing result")
    fails([SSAOp("store", (OUT, Const(1.0), None), v(0, F32))], "ssa-verifier: op #0 'store': unexpected result")
    fails([SSAOp("frobnicate", (), v(0, I32))], "unsupported operation")
    fails([SSAOp("add", (Const(1),), v(0, I32))], "expected 2 operands, got 1")
    fails([SSAOp("add", (v(0, I32), Const(1)), v(1, I32))], "%0 used before definition")
    twice = SSAOp("add", (Const(1), Const(2)), v(0, I32))
    fails([twice, SSAOp("add", (Const(1), Const(2)), v(0, I32))], "duplicate definition of %0")


def test_typing_rules():
    fails([SSAOp("add", (Const(1.0), Const(2)), v(0, I32))], "expected f32, got i32")
    fails([SSAOp("exp", (Const(1),), v(0, I32))], "exp requires f32")
    fails([SSAOp("select", (Const(1), Const(1), Const(2)), v(0, I32))], "condition must be bool")
    fails([SSAOp("and", (Const(1), Const(True)), v(0, BOOL))], "logical op requires boolean operands")
    fails([SSAOp("load", (OUT, None, Const(True)), v(0, F32))], "fallback must be convertible to f32")
    fails([SSAOp("load", (Const(1), None, None), v(0, F32))], "expected pointer")
    fails([SSAOp("addptr", (OUT, Const(1.0)), v(0, PTR_F32))], "invalid offset")
    fails([SSAOp("program_id", (), v(0, I32), {"axis": 3})], "invalid axis 3")
    fails([SSAOp("arange", (), v(0, VectorType(4, I32)), {"start": 4, "end": 4})], "invalid range")
    fails([SSAOp("zeros", (), v(0, VectorType(4, F32)), {"shape": (4,), "dtype": PTR_F32})], "invalid block dtype")
    fails([SSAOp("expand_dims", (Const(1),), v(0, I32), {"axis": 0})], "expand_dims expects block")
    ok = [
        SSAOp("arange", (), v(0, VectorType(4, I32)), {"start": 0, "end": 4}),
        SSAOp("cmp_lt", (v(0, VectorType(4, I32)), Const(2)), v(1, VectorType(4, BOOL))),
        SSAOp("addptr", (OUT, v(0, VectorType(4, I32))), v(2, VectorType(4, PTR_F32))),
        SSAOp("load", (v(2, VectorType(4, PTR_F32)), v(1, VectorType(4, BOOL)), Const(0.0)), v(3, VectorType(4, F32))),
        SSAOp("store", (v(2, VectorType(4, PTR_F32)), v(3, VectorType(4, F32)), v(1, VectorType(4, BOOL)))),
    ]
    assert verify(ok) is ok


def test_reduction_rules_and_the_cta_size_option():
    vec = VectorType(8, F32)
    program = [
        SSAOp("zeros", (), v(0, vec), {"shape": (8,), "dtype": F32}),
        SSAOp("sum", (v(0, vec),), v(1, F32)),
    ]
    verify(program)                                 # this backend: width is free of the CTA size
    verify(program, block_size=8)
    fails(program, "does not match CUDA block size 4", block_size=4)     # the reference's rule, on request
    odd = VectorType(6, F32)
    fails([SSAOp("zeros", (), v(0, odd), {"shape": (6,), "dtype": F32}), SSAOp("max", (v(0, odd),), v(1, F32))],
          "power of two")
    tile = BlockType((2, 4), F32)
    fails([SSAOp("zeros", (), v(0, tile), {"shape": (2, 4), "dtype": F32}), SSAOp("sum", (v(0, tile),), v(1, F32))],
          "reduction expects rank-1 block")
    wide = [SSAOp("arange", (), v(0, VectorType(4096, I32)), {"start": 0, "end": 4096})]
    verify(wide)
    fails(wide, "range width 4096 does not match CUDA block size 1024", block_size=1024)


def test_dot_rule():
    a, b, c = BlockType((16, 32), BF16), BlockType((32, 8), BF16), BlockType((16, 8), F32)

    def program(result_ty, rhs_ty=b):
        return [
            SSAOp("empty", (), v(0, BlockType((16, 32), F32)), {"shape": (16, 32), "dtype": F32}),
            SSAOp("dot", (SSAValue(10, a), SSAValue(11, rhs_ty), None), v(1, result_ty)),
        ]

    # operands of dot come from loads; pre-define them through a loop-free trick: params are
    # not blocks, so check the rule directly
    verifier = SSAVerifier(None)
    verifier._rule_dot(0, program(c)[1])
    with pytest.raises(CompileError, match="dot inner dimensions differ"):
        verifier._rule_dot(0, program(c, rhs_ty=a)[1])
    with pytest.raises(CompileError, match="expected block<16x8 x f32>"):
        verifier._rule_dot(0, program(BlockType((16, 8), BF16))[1])


def loop(**changes):
    fields = dict(
        index=v(0, I32), start=Const(0), stop=Param("n", I32), step=Const(1),
        carried_inputs=(Const(0),), carried_args=(v(1, I32),),
        body=[SSAOp("add", (v(1, I32), v(0, I32)), v(2, I32))],
        yields=(v(2, I32),), results=(v(3, I32),),
    )
    fields.update(changes)
    return SSAForRange(**fields)


def test_loop_regions():
    tail = SSAOp("store", (OUT, v(3, I32), None))
    verify([loop(), tail])
    fails([loop(index=v(0, F32))], "loop index must be i32, got f32")
    fails([loop(step=Const(0))], "loop step must be positive")
    fails([loop(step=Param("s", I32))], "loop step must be a constant integer")
    fails([loop(stop=Const(1.5))], "loop stop must be scalar i32")
    fails([loop(yields=(Const(1.0),))], "yield expected i32, got f32")
    fails([loop(carried_args=(v(1, F32),))], "carried arg expected i32, got f32")
    fails([loop(results=())], "mismatched yields/results")
    fails([loop(yields=(v(9, I32),))], "yield %9 used before definition")
    # body-local values are not visible after the loop
    fails([loop(), SSAOp("store", (OUT, v(2, I32), None))], "%2 used before definition")
    # outer values are visible inside
    outer = SSAOp("program_id", (), v(7, I32), {"axis": 0})
    body = [SSAOp("add", (v(1, I32), v(7, I32)), v(2, I32))]
    verify([outer, loop(body=body), tail])
