"""Structural and type verifier for SSA lists.

Checks arity, definition-before-use (with loop regions as nested scopes),
per-opcode typing and the loop-region contract.  Diagnostics have the
reference's form ``ssa-verifier: op #<i> '<opcode>': <message>``
(``src/mytriton/ssa_verification.py:52-53``) and its wording, since callers
match on them.

One deliberate difference: the reference ties block widths to the CTA size
(reduction width must equal it, ``:272-278``; arange width may not exceed it,
``:474-479``) because it runs one thread per element.  This backend gives each
thread several elements, so those two rules apply only when a ``block_size``
is passed; ``SSAVerifier(None)`` — what the JIT driver uses — skips them.
"""

from __future__ import annotations

from typing import NoReturn

from .block_shapes import broadcast_shapes
from .nodes import Const, Param
from .ssa import SSAForRange, SSAItem, SSAOp, SSAOperand, SSAValue
from .types import (
    BF16, BOOL, BYTE_WIDTH, F16, F32, FLOAT_UNARY, I32, NUMERIC, BlockType, PointerType, ScalarType, Type, element_of,
)


class CompileError(Exception):
    pass


_FOR = SSAOp("for")


class SSAVerifier:
    ARITY = {
        "program_id": 0, "num_programs": 0, "trans": 1, "arange": 0, "empty": 0, "zeros": 0, "full": 1,
        "add": 2, "sub": 2, "mul": 2, "div": 2, "rem": 2, "cmp_lt": 2, "and": 2,
        "maximum": 2, "minimum": 2, "neg": 1, "exp": 1, "not": 1,
        "addptr": 2, "load": 3, "store": 3, "atomic_add": 3, "select": 3,
        "sum": 1, "max": 1, "min": 1, "expand_dims": 1, "dot": 3, "break_unless": 1,
        **dict.fromkeys(FLOAT_UNARY, 1),
    }
    NO_RESULT = {"store", "atomic_add", "break_unless"}

    def __init__(self, block_size: int | None = None) -> None:
        self.block_size = block_size
        self._loop_depth = 0

    # -- plumbing ----------------------------------------------------------------

    def fail(self, index: int, op: SSAOp, message: str) -> NoReturn:
        raise CompileError(f"ssa-verifier: op #{index} '{op.opcode}': {message}")

    def element_type(self, ty: Type):
        return element_of(ty)

    def operand_type(self, operand: SSAOperand) -> Type | None:
        if operand is None:
            return None
        if isinstance(operand, (SSAValue, Param)):
            return operand.ty
        if isinstance(operand, Const):
            for python_type, ty in ((bool, BOOL), (int, I32), (float, F32)):
                if isinstance(operand.value, python_type):
                    return ty
        raise TypeError(f"Unknown typed operand: {operand}")

    def _need(self, index: int, op: SSAOp, operand: SSAOperand, role: str) -> Type:
        ty = self.operand_type(operand)
        if ty is None:
            self.fail(index, op, f"{role} must not be none")
        return ty

    def _result(self, index: int, op: SSAOp) -> Type:
        if op.result is None:
            self.fail(index, op, "missing result")
        return op.result.ty

    def _shaped(self, index: int, op: SSAOp, element, *types: Type) -> Type:
        shapes = [ty.shape for ty in types if isinstance(ty, BlockType)]
        if not shapes:
            return element
        try:
            return BlockType(broadcast_shapes(*shapes), element)
        except ValueError as error:
            self.fail(index, op, str(error))

    def _expect(self, index: int, op: SSAOp, actual: Type, expected: Type) -> None:
        if actual != expected:
            self.fail(index, op, f"expected {expected}, got {actual}")

    def _numeric(self, index: int, op: SSAOp, *types: Type) -> ScalarType:
        elements = [element_of(ty) for ty in types]
        if any(element not in NUMERIC for element in elements):
            self.fail(index, op, "cannot combine " + " and ".join(map(str, types)))
        return I32 if all(element == I32 for element in elements) else F32

    @staticmethod
    def _convertible(source: Type, destination) -> bool:
        have = element_of(source)
        return have == destination or (have in NUMERIC and destination in NUMERIC)

    # -- per-opcode rules --------------------------------------------------------

    def _rule_arith(self, index: int, op: SSAOp) -> None:
        lhs = self._need(index, op, op.operands[0], "lhs")
        rhs = self._need(index, op, op.operands[1], "rhs")
        element = self._numeric(index, op, lhs, rhs)
        if op.opcode == "cmp_lt":
            element = BOOL
        if op.opcode == "rem" and element != I32:
            self.fail(index, op, f"rem requires i32 operands, got {lhs} and {rhs}")
        self._expect(index, op, self._result(index, op), self._shaped(index, op, element, lhs, rhs))

    def _rule_and(self, index: int, op: SSAOp) -> None:
        lhs = self._need(index, op, op.operands[0], "lhs")
        rhs = self._need(index, op, op.operands[1], "rhs")
        if element_of(lhs) != BOOL or element_of(rhs) != BOOL:
            self.fail(index, op, "logical op requires boolean operands")
        self._expect(index, op, self._result(index, op), self._shaped(index, op, BOOL, lhs, rhs))

    def _rule_unary(self, index: int, op: SSAOp) -> None:
        operand = self._need(index, op, op.operands[0], "value")
        element = element_of(operand)
        if op.opcode == "neg" and element not in NUMERIC:
            self.fail(index, op, f"cannot negate {operand}")
        if op.opcode == "exp" and element != F32:
            self.fail(index, op, f"exp requires f32, got {operand}")
        if op.opcode == "abs" and element in (I32, F32):
            pass
        elif op.opcode in FLOAT_UNARY and element != F32:
            self.fail(index, op, f"{op.opcode} requires f32, got {operand}")
        if op.opcode == "not" and element != BOOL:
            self.fail(index, op, f"not requires a boolean, got {operand}")
        self._expect(index, op, self._result(index, op), operand)

    def _rule_addptr(self, index: int, op: SSAOp) -> None:
        base = self._need(index, op, op.operands[0], "base")
        offset = self._need(index, op, op.operands[1], "offset")
        pointer = element_of(base)
        if not isinstance(pointer, PointerType):
            self.fail(index, op, f"invalid base {base}")
        if element_of(offset) != I32:
            self.fail(index, op, f"invalid offset {offset}")
        self._expect(
            index, op, self._result(index, op), self._shaped(index, op, pointer, base, offset)
        )

    def _mask(self, index: int, op: SSAOp, mask: SSAOperand) -> Type:
        ty = self._need(index, op, mask, "mask")
        if element_of(ty) != BOOL:
            self.fail(index, op, f"mask must be bool, got {ty}")
        return ty

    def _rule_load(self, index: int, op: SSAOp) -> None:
        ptr, mask, other = op.operands
        ptr_ty = self._need(index, op, ptr, "pointer")
        pointer = element_of(ptr_ty)
        result_ty = self._result(index, op)
        if not isinstance(pointer, PointerType):
            self.fail(index, op, f"expected pointer, got {ptr_ty}")
        shaped = [ptr_ty]
        if mask is not None:
            shaped.append(self._mask(index, op, mask))
        if other is not None:
            other_ty = self._need(index, op, other, "fallback")
            if not self._convertible(other_ty, pointer.element):
                self.fail(
                    index, op,
                    f"fallback must be convertible to {pointer.element}, got {other_ty}",
                )
            shaped.append(other_ty)
        self._expect(index, op, result_ty, self._shaped(index, op, pointer.element, *shaped))

    def _rule_store(self, index: int, op: SSAOp) -> None:
        ptr, value, mask = op.operands
        ptr_ty = self._need(index, op, ptr, "pointer")
        value_ty = self._need(index, op, value, "value")
        pointer = element_of(ptr_ty)
        if not isinstance(pointer, PointerType):
            self.fail(index, op, f"expected pointer, got {ptr_ty}")
        if not self._convertible(value_ty, pointer.element):
            self.fail(
                index, op,
                f"stored value must be convertible to {pointer.element}, got {value_ty}",
            )
        if op.opcode == "atomic_add" and pointer.element not in (F32, I32):
            self.fail(index, op, f"atomic_add needs an f32 or i32 array, got {ptr_ty}")
        shaped = [ptr_ty, value_ty]
        if mask is not None:
            shaped.append(self._mask(index, op, mask))
        self._shaped(index, op, pointer.element, *shaped)

    def _rule_select(self, index: int, op: SSAOp) -> None:
        roles = ("condition", "true value", "false value")
        cond, yes, no = (self._need(index, op, x, r) for x, r in zip(op.operands, roles))
        result_ty = self._result(index, op)
        if element_of(cond) != BOOL:
            self.fail(index, op, f"condition must be bool, got {cond}")
        element = self._numeric(index, op, yes, no)
        self._expect(index, op, result_ty, self._shaped(index, op, element, cond, yes, no))

    def _rule_reduce(self, index: int, op: SSAOp) -> None:
        operand = self._need(index, op, op.operands[0], "value")
        result_ty = self._result(index, op)
        if isinstance(operand, BlockType) and operand.rank == 2 and "axis" in op.attrs:
            axis = op.attrs["axis"]
            if axis not in (0, 1):
                self.fail(index, op, f"invalid axis {axis}")
            if operand.element not in (I32, F32):
                self.fail(index, op, f"cannot reduce elements of type {operand.element}")
            self._expect(index, op, result_ty, BlockType((operand.shape[1 - axis],), operand.element))
            return
        if not isinstance(operand, BlockType) or operand.rank != 1:
            self.fail(index, op, f"reduction expects rank-1 block, got {operand}")
        if self.block_size is not None and operand.size != self.block_size:
            self.fail(
                index, op,
                f"reduction width {operand.size} does not match "
                f"CUDA block size {self.block_size}",
            )
        if operand.size & (operand.size - 1):
            self.fail(index, op, f"reduction width must be a power of two, got {operand.size}")
        if operand.element not in (I32, F32):
            self.fail(index, op, f"cannot reduce elements of type {operand.element}")
        self._expect(index, op, result_ty, operand.element)

    def _rule_trans(self, index: int, op: SSAOp) -> None:
        operand = self._need(index, op, op.operands[0], "value")
        if not isinstance(operand, BlockType) or operand.rank != 2:
            self.fail(index, op, f"trans expects a rank-2 block, got {operand}")
        self._expect(index, op, self._result(index, op),
                     BlockType((operand.shape[1], operand.shape[0]), operand.element))

    def _rule_expand_dims(self, index: int, op: SSAOp) -> None:
        operand = self._need(index, op, op.operands[0], "value")
        result_ty = self._result(index, op)
        axis = op.attrs.get("axis")
        if not isinstance(operand, BlockType):
            self.fail(index, op, f"expand_dims expects block, got {operand}")
        if type(axis) is not int or not 0 <= axis <= operand.rank:
            self.fail(index, op, f"invalid axis {axis}")
        dims = list(operand.shape)
        dims.insert(axis, 1)
        self._expect(index, op, result_ty, BlockType(tuple(dims), operand.element))

    def _rule_program_id(self, index: int, op: SSAOp) -> None:
        if op.attrs.get("axis") not in (0, 1, 2):
            self.fail(index, op, f"invalid axis {op.attrs.get('axis')}")
        self._expect(index, op, self._result(index, op), I32)

    def _rule_arange(self, index: int, op: SSAOp) -> None:
        start, end = op.attrs.get("start"), op.attrs.get("end")
        if type(start) is not int or type(end) is not int:
            self.fail(index, op, "arange start and end must be integers")
        width = end - start
        if width <= 0:
            self.fail(index, op, f"invalid range [{start}, {end})")
        self._expect(index, op, self._result(index, op), BlockType((width,), I32))
        if self.block_size is not None and width > self.block_size:
            self.fail(
                index, op,
                f"range width {width} does not match CUDA block size {self.block_size}",
            )

    def _rule_constructor(self, index: int, op: SSAOp) -> None:
        shape, dtype = op.attrs.get("shape"), op.attrs.get("dtype")
        well_formed = (
            isinstance(shape, tuple)
            and len(shape) > 0
            and all(type(dim) is int and dim > 0 for dim in shape)
        )
        if not well_formed:
            self.fail(index, op, f"invalid block shape {shape}")
        if dtype not in (BOOL, I32, F32):
            self.fail(index, op, f"invalid block dtype {dtype}")
        self._expect(index, op, self._result(index, op), BlockType(shape, dtype))
        if op.opcode == "full":
            fill = self._need(index, op, op.operands[0], "fill value")
            if isinstance(fill, BlockType):
                self.fail(index, op, f"fill value must be scalar, got {fill}")
            if not self._convertible(fill, dtype):
                self.fail(index, op, f"fill value must be convertible to {dtype}, got {fill}")

    def _rule_dot(self, index: int, op: SSAOp) -> None:
        lhs = self._need(index, op, op.operands[0], "lhs")
        rhs = self._need(index, op, op.operands[1], "rhs")
        for ty in (lhs, rhs):
            if not isinstance(ty, BlockType) or ty.rank != 2 or ty.element not in (F32, BF16, F16) + BYTE_WIDTH:
                self.fail(index, op, f"dot expects rank-2 f32/bf16/f16/fp8 blocks, got {ty}")
        if lhs.element != rhs.element:
            self.fail(index, op, f"dot operand element types differ: {lhs} and {rhs}")
        if lhs.shape[1] != rhs.shape[0]:
            self.fail(index, op, f"dot inner dimensions differ: {lhs} and {rhs}")
        expected = BlockType((lhs.shape[0], rhs.shape[1]), F32)
        acc = self.operand_type(op.operands[2])
        if acc is not None and acc != expected:
            self.fail(index, op, f"dot accumulator must be {expected}, got {acc}")
        self._expect(index, op, self._result(index, op), expected)

    def _rule_break_unless(self, index: int, op: SSAOp) -> None:
        if self._loop_depth == 0:
            self.fail(index, op, "break_unless outside a loop body")
        condition = self._need(index, op, op.operands[0], "condition")
        if condition != BOOL:
            self.fail(index, op, f"condition must be a scalar boolean, got {condition}")

    RULES = {
        "break_unless": _rule_break_unless,
        **dict.fromkeys(("add", "sub", "mul", "div", "rem", "cmp_lt", "maximum", "minimum"), _rule_arith),
        "and": _rule_and,
        "neg": _rule_unary, "exp": _rule_unary, "not": _rule_unary,
        **dict.fromkeys(FLOAT_UNARY, _rule_unary),
        "addptr": _rule_addptr, "load": _rule_load, "store": _rule_store, "atomic_add": _rule_store,
        "select": _rule_select,
        "sum": _rule_reduce, "max": _rule_reduce, "min": _rule_reduce,
        "expand_dims": _rule_expand_dims, "trans": _rule_trans, "program_id": _rule_program_id, "num_programs": _rule_program_id,
        "arange": _rule_arange, "dot": _rule_dot,
        **dict.fromkeys(("empty", "full", "zeros"), _rule_constructor),
    }

    # the reference's method names, for code that calls one rule directly
    check_binary_numeric = _rule_arith
    check_binary_bool = _rule_and
    check_unary = _rule_unary
    check_addptr = _rule_addptr
    check_load = _rule_load
    check_store = _rule_store
    check_select = _rule_select
    check_reduction = _rule_reduce
    check_expand_dims = _rule_expand_dims
    check_program_id = _rule_program_id
    check_arange = _rule_arange
    check_block_constructor = _rule_constructor
    check_dot = _rule_dot

    # -- loops -------------------------------------------------------------------

    def _bound(self, index: int, operand: SSAOperand, role: str, defined: set[int]) -> None:
        if isinstance(operand, SSAValue) and operand.id not in defined:
            self.fail(index, _FOR, f"{role} {operand} used before definition")
        ty = self._need(index, _FOR, operand, role)
        if ty != I32:
            self.fail(index, _FOR, f"{role} must be scalar i32, got {ty}")

    def _fresh(self, index: int, value: SSAValue, role: str, defined: set[int]) -> None:
        if value.id in defined:
            self.fail(index, _FOR, f"duplicate definition of {role} {value}")
        defined.add(value.id)

    def check_for_range(self, index: int, loop: SSAForRange, defined: set[int]) -> None:
        self._bound(index, loop.start, "loop start", defined)
        self._bound(index, loop.stop, "loop stop", defined)
        self._bound(index, loop.step, "loop step", defined)
        if loop.index.ty != I32:
            self.fail(index, _FOR, f"loop index must be i32, got {loop.index.ty}")
        if not isinstance(loop.step, Const) or type(loop.step.value) is not int:
            self.fail(index, _FOR, "loop step must be a constant integer")
        if loop.step.value <= 0:
            self.fail(index, _FOR, "loop step must be positive")
        if len(loop.carried_inputs) != len(loop.carried_args):
            self.fail(index, _FOR, "mismatched carried inputs/args")
        if len(loop.yields) != len(loop.results):
            self.fail(index, _FOR, "mismatched yields/results")
        if len(loop.carried_inputs) != len(loop.results):
            self.fail(index, _FOR, "mismatched carried inputs/results")

        scope = set(defined)
        self._fresh(index, loop.index, "loop index", scope)
        for initial, arg in zip(loop.carried_inputs, loop.carried_args, strict=True):
            if isinstance(initial, SSAValue) and initial.id not in defined:
                self.fail(index, _FOR, f"carried input {initial} used before definition")
            initial_ty = self._need(index, _FOR, initial, "carried input")
            if arg.ty != initial_ty:
                self.fail(index, _FOR, f"carried arg expected {initial_ty}, got {arg.ty}")
            self._fresh(index, arg, "carried argument", scope)

        self._loop_depth += 1
        try:
            self._verify_ops(loop.body, scope)
        finally:
            self._loop_depth -= 1

        rows = zip(loop.carried_inputs, loop.carried_args, loop.yields, loop.results, strict=True)
        for initial, arg, yielded, result in rows:
            if isinstance(yielded, SSAValue) and yielded.id not in scope:
                self.fail(index, _FOR, f"yield {yielded} used before definition")
            initial_ty = self._need(index, _FOR, initial, "carried input")
            yield_ty = self._need(index, _FOR, yielded, "yield")
            if yield_ty != arg.ty:
                self.fail(index, _FOR, f"yield expected {arg.ty}, got {yield_ty}")
            if result.ty != yield_ty:
                self.fail(index, _FOR, f"loop result expected {yield_ty}, got {result.ty}")
            if result.ty != initial_ty:
                self.fail(
                    index, _FOR, f"loop result expected carried type {initial_ty}, got {result.ty}"
                )
        for result in loop.results:
            self._fresh(index, result, "loop result", scope)
            defined.add(result.id)

    # -- driver ------------------------------------------------------------------

    def verify(self, ops: list[SSAItem]) -> list[SSAItem]:
        self._verify_ops(ops, set())
        return ops

    def _verify_ops(self, ops: list[SSAItem], defined: set[int]) -> None:
        for index, op in enumerate(ops):
            if isinstance(op, SSAForRange):
                self.check_for_range(index, op, defined)
                continue
            arity = self.ARITY.get(op.opcode)
            if arity is None:
                self.fail(index, op, "unsupported operation")
            if len(op.operands) != arity:
                self.fail(index, op, f"expected {arity} operands, got {len(op.operands)}")
            if op.opcode in self.NO_RESULT:
                if op.result is not None:
                    self.fail(index, op, "unexpected result")
            elif op.result is None:
                self.fail(index, op, "missing result")
            for operand in op.operands:
                if isinstance(operand, SSAValue) and operand.id not in defined:
                    self.fail(index, op, f"{operand} used before definition")
            self.RULES[op.opcode](self, index, op)
            if op.result is not None:
                if op.result.id in defined:
                    self.fail(index, op, f"duplicate definition of {op.result}")
                defined.add(op.result.id)
