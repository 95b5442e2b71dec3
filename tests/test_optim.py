"""Optimisation passes (CPU): folding rules with their float caveats, CSE, DCE, the
pass manager, and the region-aware mode that goes beyond the reference."""

import math

import numpy as np
import pytest

from mytriton_b200 import kernels as corpus
from mytriton_b200.nodes import Const, Param
from mytriton_b200.optim import ConstantFoldPass, CSEPass, DCEPass, PassManager
from mytriton_b200.ssa import SSAForRange, SSAOp, SSAPrinter, SSAValue
from mytriton_b200.ssa_verification import CompileError, SSAVerifier
from mytriton_b200.types import BOOL, F32, I32, PTR_F32

OUT = Param("out", PTR_F32)
X = Param("x", F32)
N = Param("n", I32)


def v(i, ty):
    return SSAValue(i, ty)


def store(value):
    return SSAOp("store", (OUT, value, None))


def text(ops):
    return SSAPrinter().print_ops(ops)


def test_constant_folding_and_integer_semantics():
    ops = [
        SSAOp("mul", (Const(6), Const(7)), v(0, I32)),
        SSAOp("div", (Const(-7), Const(2)), v(1, I32)),            # C division: toward zero
        SSAOp("add", (v(0, I32), v(1, I32)), v(2, I32)),
        SSAOp("cmp_lt", (Const(1), Const(2)), v(3, BOOL)),
        SSAOp("select", (v(3, BOOL), v(2, I32), Const(0)), v(4, I32)),
        store(v(4, I32)),
    ]
    assert text(ConstantFoldPass().run(ops)) == "store out, 39, none"


def test_float_identities_are_conservative():
    ops = [
        SSAOp("add", (X, Const(0.0)), v(0, F32)),                  # kept: x + 0.0 changes -0.0
        SSAOp("mul", (v(0, F32), Const(1.0)), v(1, F32)),          # folded
        SSAOp("div", (v(1, F32), Const(1)), v(2, F32)),            # folded
        SSAOp("add", (N, Const(0)), v(3, I32)),                    # folded for integers
        SSAOp("select", (Param("c", BOOL), v(2, F32), v(2, F32)), v(4, F32)),   # same arms
        store(v(4, F32)),
        store(v(3, I32)),
    ]
    assert text(ConstantFoldPass().run(ops)) == "%0 = add x, 0.0 : f32\nstore out, %0, none\nstore out, n, none"


def test_extrema_and_nan_signed_zero_folding():
    fold = ConstantFoldPass()

    def folded(opcode, lhs, rhs):
        (op,) = fold.run([SSAOp(opcode, (Const(lhs), Const(rhs)), v(0, F32)), store(v(0, F32))])[-1:]
        return op.operands[1].value

    assert math.isnan(folded("maximum", float("nan"), 2.0)) and math.isnan(folded("minimum", 2.0, float("nan")))
    assert math.copysign(1, folded("maximum", 0.0, -0.0)) == -1     # ties return the right operand
    assert math.copysign(1, folded("minimum", -0.0, 0.0)) == 1
    assert folded("maximum", 3.0, 2.0) == 3.0 and folded("minimum", 3.0, 2.0) == 2.0
    # division by zero is left for the device
    kept = fold.run([SSAOp("div", (Const(1), Const(0)), v(0, I32)), store(v(0, I32))])
    assert kept[0].opcode == "div"


def test_cse_distinguishes_signed_zero_and_types():
    ops = [
        SSAOp("add", (X, Const(0.0)), v(0, F32)),
        SSAOp("add", (X, Const(-0.0)), v(1, F32)),                 # different constant (hex key)
        SSAOp("add", (X, Const(0.0)), v(2, F32)),                  # same as %0
        SSAOp("load", (OUT, None, None), v(3, F32)),
        SSAOp("load", (OUT, None, None), v(4, F32)),               # loads are never merged
        store(v(0, F32)), store(v(1, F32)), store(v(2, F32)), store(v(3, F32)), store(v(4, F32)),
    ]
    out = CSEPass().run(ops)
    assert [op.opcode for op in out].count("add") == 2 and [op.opcode for op in out].count("load") == 2
    assert out[6].operands[1] == v(0, F32)                          # third store now reads %0


def test_dce_keeps_only_what_stores_need():
    ops = [
        SSAOp("add", (X, Const(1.0)), v(0, F32)),
        SSAOp("mul", (X, Const(2.0)), v(1, F32)),                  # dead
        store(v(0, F32)),
    ]
    assert text(DCEPass().run(ops)) == "%0 = add x, 1.0 : f32\nstore out, %0, none"


def test_pass_manager_verifies_after_every_pass():
    class Breaks:
        def run(self, ops):
            return [SSAOp("add", (v(99, F32), Const(1.0)), v(0, F32)), *ops]

    with pytest.raises(CompileError, match="%99 used before definition"):
        PassManager([Breaks()], SSAVerifier(None)).run([store(Const(1.0))])


def looped_program():
    kernel = corpus.matmul_runtime_k_kernel
    kernel.clear_cache()
    a = np.zeros((5, 3), np.float32)
    _, ssa_ops, _ = kernel[(2, 1)](a, np.zeros((3, 7), np.float32), np.zeros((5, 7), np.float32),
                                   5, 7, 3, BM=4, BN=8)
    return ssa_ops


def test_loops_are_left_alone_by_default_and_optimised_on_request():
    ssa_ops = looped_program()
    passes = [ConstantFoldPass(), CSEPass(), DCEPass()]
    untouched = PassManager(passes, SSAVerifier(None)).run(ssa_ops)
    assert untouched is ssa_ops                                     # the reference's behaviour
    optimised = PassManager(passes, SSAVerifier(None), region_aware=True).run(ssa_ops)
    before = text(ssa_ops)
    after = text(optimised)
    assert before.count("cmp_lt") == 4 and after.count("cmp_lt") == 4   # body values do not leak out
    loop = next(op for op in optimised if isinstance(op, SSAForRange))
    assert len(loop.body) <= len(next(op for op in ssa_ops if isinstance(op, SSAForRange)).body)
    SSAVerifier(None).verify(optimised)


def test_region_aware_cse_merges_inside_a_body_and_dce_drops_dead_loops():
    body = [
        SSAOp("add", (v(1, I32), N), v(2, I32)),
        SSAOp("add", (v(1, I32), N), v(3, I32)),                   # duplicate inside the body
        SSAOp("add", (v(2, I32), v(3, I32)), v(4, I32)),
    ]
    live = SSAForRange(v(0, I32), Const(0), N, Const(1), (Const(0),), (v(1, I32),), body, (v(4, I32),), (v(5, I32),))
    dead = SSAForRange(v(6, I32), Const(0), N, Const(1), (Const(0),), (v(7, I32),),
                       [SSAOp("add", (v(7, I32), Const(1)), v(8, I32))], (v(8, I32),), (v(9, I32),))
    program = [live, dead, store(v(5, I32))]
    out = PassManager([CSEPass(), DCEPass()], SSAVerifier(None), region_aware=True).run(program)
    assert len(out) == 2                                            # the unused loop is gone
    assert [op.opcode for op in out[0].body] == ["add", "add"]
    assert out[0].body[1].operands == (v(2, I32), v(2, I32))


def test_identity_folds_never_change_a_type():
    """`i32 * 1.0` is f32: the operand cannot stand in for the result (the reference
    folds it anyway and then trips its own verifier)."""
    from mytriton_b200.types import VectorType

    lanes = v(0, VectorType(8, I32))
    ops = [
        SSAOp("arange", (), lanes, {"start": 0, "end": 8}),
        SSAOp("mul", (lanes, Const(1.0)), v(1, VectorType(8, F32))),
        SSAOp("mul", (v(1, VectorType(8, F32)), Const(3)), v(2, VectorType(8, F32))),
        SSAOp("mul", (lanes, Const(1)), v(3, VectorType(8, I32))),
        SSAOp("addptr", (OUT, v(3, VectorType(8, I32))), v(4, VectorType(8, PTR_F32))),
        SSAOp("store", (v(4, VectorType(8, PTR_F32)), v(2, VectorType(8, F32)), None)),
    ]
    out = PassManager([ConstantFoldPass(), CSEPass(), DCEPass()], SSAVerifier(None)).run(ops)
    assert [op.opcode for op in out] == ["arange", "mul", "mul", "addptr", "store"]
    assert out[3].operands[1] == lanes                   # the i32 * 1 did fold


def test_select_folds_only_to_an_arm_of_the_result_type():
    """select(const, block, scalar) and select(block_cond, s, s) have block results; the
    scalar arm cannot replace them (a consumer's recorded type would no longer verify)."""
    from mytriton_b200.types import VectorType

    lanes, scalar = v(0, VectorType(8, I32)), Param("s", F32)
    block_f = VectorType(8, F32)
    ops = [
        SSAOp("arange", (), lanes, {"start": 0, "end": 8}),
        SSAOp("cmp_lt", (lanes, Const(3)), v(1, VectorType(8, BOOL))),
        SSAOp("select", (Const(False), lanes, scalar), v(2, block_f)),          # scalar arm, block result
        SSAOp("select", (v(1, VectorType(8, BOOL)), scalar, scalar), v(3, block_f)),
        SSAOp("add", (v(2, block_f), v(3, block_f)), v(4, block_f)),
        SSAOp("select", (Const(True), v(4, block_f), scalar), v(5, block_f)),   # same type: folds
        SSAOp("addptr", (OUT, lanes), v(6, VectorType(8, PTR_F32))),
        SSAOp("store", (v(6, VectorType(8, PTR_F32)), v(5, block_f), None)),
    ]
    out = PassManager([ConstantFoldPass(), CSEPass(), DCEPass()], SSAVerifier(None)).run(ops)
    assert [op.opcode for op in out].count("select") == 2
    assert out[-1].operands[1] == v(4, block_f)


# ---------------------------------------------------------------- loop-invariant motion


def test_loop_invariant_motion_moves_pure_operations_and_nothing_else():
    from mytriton_b200.optim import LoopInvariantMotionPass

    body = [
        SSAOp("mul", (N, Const(4)), v(2, I32)),                    # invariant
        SSAOp("add", (v(2, I32), v(0, I32)), v(3, I32)),           # uses the index
        SSAOp("div", (N, N), v(4, I32)),                           # integer division by a run-time value
        SSAOp("div", (N, Const(2)), v(5, I32)),                    # by a non-zero constant: may move
        SSAOp("add", (v(1, I32), v(5, I32)), v(6, I32)),           # uses the carried argument
        SSAOp("add", (v(6, I32), v(4, I32)), v(7, I32)),
        SSAOp("add", (v(7, I32), v(3, I32)), v(8, I32)),
    ]
    loop = SSAForRange(v(0, I32), Const(0), N, Const(1), (Const(0),), (v(1, I32),), body, (v(8, I32),), (v(9, I32),))
    out = LoopInvariantMotionPass().run([loop, store(v(9, I32))])
    assert [op.result.id for op in out[:2]] == [2, 5]
    assert [op.result.id for op in out[2].body] == [3, 4, 6, 7, 8]
    SSAVerifier(None).verify(out)


def test_loop_invariant_motion_leaves_a_whole_nest():
    from mytriton_b200.optim import LoopInvariantMotionPass

    inner_body = [
        SSAOp("mul", (N, Const(3)), v(4, I32)),                    # invariant in both loops
        SSAOp("mul", (v(0, I32), Const(2)), v(5, I32)),            # depends on the outer index only
        SSAOp("add", (v(4, I32), v(5, I32)), v(6, I32)),
        SSAOp("add", (v(3, I32), v(6, I32)), v(7, I32)),
    ]
    inner = SSAForRange(v(2, I32), Const(0), N, Const(1), (v(1, I32),), (v(3, I32),), inner_body,
                        (v(7, I32),), (v(8, I32),))
    outer = SSAForRange(v(0, I32), Const(0), N, Const(1), (Const(0),), (v(1, I32),), [inner],
                        (v(8, I32),), (v(9, I32),))
    out = LoopInvariantMotionPass().run([outer, store(v(9, I32))])
    assert [op.result.id for op in out[:1]] == [4]                 # out of both loops
    outer_body = out[1].body
    assert [op.result.id for op in outer_body[:2]] == [5, 6]       # out of the inner loop
    assert [op.result.id for op in outer_body[2].body] == [7]
    SSAVerifier(None).verify(out)


def test_the_code_generator_gets_hoisted_addresses_and_callers_get_the_reference_ssa():
    """tests/test_ast_runtime_loop.py:447-459 of the reference pins `v4*K` and both masks
    inside the loop; here they are computed once in front of it, while the SSA handed back
    is still the untouched one."""
    kernel = corpus.matmul_runtime_k_kernel
    kernel.clear_cache()
    args = (np.zeros((5, 3), np.float32), np.zeros((3, 7), np.float32), np.zeros((5, 7), np.float32), 5, 7, 3)
    _, ssa_ops, src = kernel[(2, 1)](*args, BM=4, BN=8)
    loop = next(op for op in ssa_ops if isinstance(op, SSAForRange))
    assert sum(op.opcode == "cmp_lt" for op in loop.body) == 2      # reference SSA: masks in the body
    head, _, tail = src.partition("for (int v11 = 0; v11 < K;")
    assert tail and "* K)" in head and "* K)" not in tail
    assert head.count(" < M)") == 1 and head.count(" < N)") == 1 and " < M)" not in tail.split("}\n    int")[0]
    kernel.clear_cache()
    _, _, plain = kernel[(2, 1)](*args, BM=4, BN=8, loop_passes=False)
    assert "* K)" in plain.partition("for (int v11 = 0; v11 < K;")[2]
