"""SSA optimisation passes: constant folding, common-subexpression elimination,
dead-code elimination, and the pass manager that re-verifies after each pass.

Folding rules and their caution about floats are the reference's
(``src/mytriton/optim.py:50-172``): ``x+0``/``x-0`` fold for integers only (so
``-0.0`` survives), ``x*1`` and ``x/1`` fold, ``select`` with a constant
condition or identical arms folds, i32 division truncates toward zero, and
float extrema propagate NaN and return the right operand on ties.  CSE keys
floats by their hex form so ``0.0`` and ``-0.0`` stay distinct (``:20-24``).

The reference leaves a kernel untouched as soon as it contains a runtime loop
(``:268-277``), so its generated loops re-derive addresses and masks on every
iteration.  These passes work inside loops too: bodies are folded and CSE'd in a
nested scope, liveness flows through ``yield``s, and ``LoopInvariantMotionPass``
moves operations that do not depend on the iteration in front of the loop.  The
compiler keeps two programs: the SSA it hands back to callers is produced the
reference's way (``PassManager`` without ``region_aware``), the SSA it hands to
the code generator is produced by ``codegen_pipeline``.
"""

from __future__ import annotations

import math
from collections.abc import Mapping

from .nodes import Const, Param
from .ssa import SSAForRange, SSAOp, SSAOperand, SSAValue
from .types import BOOL, F32, FLOAT_UNARY, I32, element_of


def const_key(value: object) -> tuple[object, ...]:
    return (float, value.hex()) if isinstance(value, float) else (type(value), value)


def operand_key(operand: SSAOperand) -> tuple[object, ...]:
    if operand is None:
        return ("none",)
    if isinstance(operand, SSAValue):
        return ("ssa", operand.id)
    if isinstance(operand, Param):
        return ("param", operand.name, operand.ty)
    if isinstance(operand, Const):
        return ("const", *const_key(operand.value))
    raise TypeError(f"Unknown operand: {operand}")


def resolve_operand(operand: SSAOperand, replacements: Mapping[int, SSAOperand]) -> SSAOperand:
    while isinstance(operand, SSAValue) and operand.id in replacements:
        operand = replacements[operand.id]
    return operand


def _rewrite_loop(loop: SSAForRange, replacements, body) -> SSAForRange:
    fix = lambda operand: resolve_operand(operand, replacements)  # noqa: E731
    return SSAForRange(
        index=loop.index,
        start=fix(loop.start),
        stop=fix(loop.stop),
        step=fix(loop.step),
        carried_inputs=tuple(map(fix, loop.carried_inputs)),
        carried_args=loop.carried_args,
        body=body,
        yields=tuple(map(fix, loop.yields)),
        results=loop.results,
    )


def _with_operands(op: SSAOp, replacements) -> SSAOp:
    operands = tuple(resolve_operand(x, replacements) for x in op.operands)
    return SSAOp(op.opcode, operands, op.result, dict(op.attrs))


class ConstantFoldPass:
    def scalar_type(self, ty):
        return element_of(ty)

    def normalize(self, value, ty):
        element = element_of(ty)
        if element == F32:
            return float(value)
        if element == I32:
            return int(value)
        if element == BOOL:
            return bool(value)
        raise TypeError(f"Cannot create constant of type {element}")

    def extremum(self, opcode, lhs, rhs, ty):
        if element_of(ty) == F32:
            lhs, rhs = float(lhs), float(rhs)
            if math.isnan(lhs):
                return lhs
            if math.isnan(rhs):
                return rhs
        if opcode == "maximum":
            return lhs if lhs > rhs else rhs
        return lhs if lhs < rhs else rhs

    def _evaluate(self, op: SSAOp, values: list):
        integer = element_of(op.result.ty) == I32
        code = op.opcode
        if code == "add":
            return values[0] + values[1]
        if code == "sub":
            return values[0] - values[1]
        if code == "mul":
            return values[0] * values[1]
        if code == "div":
            quotient = values[0] / values[1]
            return int(quotient) if integer else quotient
        if code == "rem":
            return int(math.fmod(values[0], values[1]))      # C remainder: the dividend's sign
        if code == "cmp_lt":
            return values[0] < values[1]
        if code == "neg":
            return -values[0]
        if code == "not":
            return not values[0]
        if code == "exp":
            return math.exp(values[0])
        if code in ("maximum", "minimum"):
            return self.extremum(code, values[0], values[1], op.result.ty)
        return None

    def fold(self, op: SSAOp) -> SSAOperand:
        """Return the operand that can stand in for ``op.result``, or None."""
        operands = op.operands
        if op.opcode == "select":
            condition, yes, no = operands
            if isinstance(condition, Const):
                chosen = yes if condition.value else no
            else:
                chosen = yes if operand_key(yes) == operand_key(no) else None
            # the chosen arm may be narrower than the result (a scalar arm of a select whose
            # other arm or condition is a block): then it cannot stand in for it
            return chosen if chosen is not None and _has_type(chosen, op.result.ty) else None
        if op.opcode == "dot":
            return None
        if len(operands) == 2 and isinstance(operands[1], Const):
            lhs, rhs = operands
            # an identity may only stand in for the result if it has the result's type
            # (`i32_block * 1.0` is an f32 block: the reference folds it to the i32
            # operand and then fails its own verifier)
            same_type = getattr(lhs, "ty", None) == op.result.ty
            additive = op.opcode in ("add", "sub") and element_of(op.result.ty) == I32
            if additive and rhs.value == 0 and same_type:
                return lhs
            if op.opcode in ("mul", "div") and rhs.value == 1 and same_type:
                return lhs
        if not operands or not all(isinstance(x, Const) for x in operands):
            return None
        try:
            value = self._evaluate(op, [x.value for x in operands])
        except (ArithmeticError, OverflowError, ValueError):     # e.g. a constant division by zero
            return None
        return None if value is None else Const(self.normalize(value, op.result.ty))

    def run(self, ops, replacements: dict[int, SSAOperand] | None = None):
        replacements = {} if replacements is None else replacements
        kept = []
        for op in ops:
            if isinstance(op, SSAForRange):
                kept.append(self._run_loop(op, replacements))
                continue
            candidate = _with_operands(op, replacements)
            folded = self.fold(candidate) if candidate.result is not None else None
            if folded is None:
                kept.append(candidate)
            else:
                replacements[candidate.result.id] = folded
        return kept

    def _run_loop(self, loop: SSAForRange, replacements) -> SSAForRange:
        body = self.run(loop.body, replacements)
        return _rewrite_loop(loop, replacements, body)


def _has_type(operand: SSAOperand, ty) -> bool:
    if isinstance(operand, Const):
        python_type = {BOOL: bool, I32: int, F32: float}.get(ty)
        return python_type is not None and type(operand.value) is python_type
    return getattr(operand, "ty", None) == ty


class CSEPass:
    PURE_OPS = {
        "program_id", "num_programs", "arange", "full", "zeros", "add", "sub", "mul", "div", "rem", "cmp_lt",
        "neg", "not", "exp", "maximum", "minimum", "addptr", "select", "and", "expand_dims", "trans",
        *FLOAT_UNARY,
    }

    def operand_key(self, operand):
        return operand_key(operand)

    def run(self, ops, replacements=None, available=None):
        replacements = {} if replacements is None else replacements
        available = {} if available is None else available
        kept = []
        for op in ops:
            if isinstance(op, SSAForRange):
                # the body sees outer expressions; what it defines stays inside
                body = self.run(op.body, replacements, dict(available))
                kept.append(_rewrite_loop(op, replacements, body))
                continue
            candidate = _with_operands(op, replacements)
            result = candidate.result
            if result is None or op.opcode not in self.PURE_OPS:
                kept.append(candidate)
                continue
            key = (
                op.opcode,
                tuple(operand_key(x) for x in candidate.operands),
                tuple(sorted(op.attrs.items())),
                result.ty,
            )
            earlier = available.get(key)
            if earlier is None:
                available[key] = result
                kept.append(candidate)
            else:
                replacements[result.id] = earlier
        return kept


class DCEPass:
    SIDE_EFFECTS = {"store", "atomic_add", "break_unless"}

    def run(self, ops, live: set[int] | None = None):
        live = set() if live is None else live
        kept = []
        for op in reversed(ops):
            if isinstance(op, SSAForRange):
                survivor = self._run_loop(op, live)
                if survivor is not None:
                    kept.append(survivor)
                continue
            wanted = op.opcode in self.SIDE_EFFECTS or (
                op.result is not None and op.result.id in live
            )
            if not wanted:
                continue
            if op.result is not None:
                live.discard(op.result.id)
            live.update(x.id for x in op.operands if isinstance(x, SSAValue))
            kept.append(op)
        kept.reverse()
        return kept

    @staticmethod
    def _has_effect(ops) -> bool:
        for op in ops:
            if isinstance(op, SSAForRange):
                if DCEPass._has_effect(op.body):
                    return True
            elif op.opcode in DCEPass.SIDE_EFFECTS:
                return True
        return False

    def _run_loop(self, loop: SSAForRange, live: set[int]):
        results_used = any(result.id in live for result in loop.results)
        if not results_used and not self._has_effect(loop.body):
            return None
        # Carried slots are kept as a group: every yield stays live.  A body value
        # may feed itself through a carried argument, so iterate to a fixed point.
        inner = {x.id for x in loop.yields if isinstance(x, SSAValue)}
        body = self.run(loop.body, inner)
        for result in loop.results:
            live.discard(result.id)
        inner -= {loop.index.id, *(arg.id for arg in loop.carried_args)}
        live |= inner
        for operand in (loop.start, loop.stop, loop.step, *loop.carried_inputs):
            if isinstance(operand, SSAValue):
                live.add(operand.id)
        return SSAForRange(
            loop.index, loop.start, loop.stop, loop.step, loop.carried_inputs,
            loop.carried_args, body, loop.yields, loop.results,
        )


class LoopInvariantMotionPass:
    """Moves pure operations out of run-time loops when none of their operands is
    defined by the loop (its index, its carried arguments, or a value computed from
    them).  Inner loops are emptied first, so an operation can travel out of a whole
    nest.  Loads stay where they are (a store in the loop may alias them), and so does
    an integer division whose divisor is not a non-zero constant: in front of a loop
    that runs zero times it would be evaluated where the program never did."""

    MOVABLE = CSEPass.PURE_OPS

    def run(self, ops):
        out = []
        for op in ops:
            if isinstance(op, SSAForRange):
                moved, loop = self._split(op)
                out.extend(moved)
                out.append(loop)
            else:
                out.append(op)
        return out

    @staticmethod
    def _safe_anywhere(op: SSAOp) -> bool:
        if op.opcode in ("div", "rem") and element_of(op.result.ty) == I32:
            divisor = op.operands[1]
            return isinstance(divisor, Const) and divisor.value != 0
        return True

    def _split(self, loop: SSAForRange):
        body = self.run(loop.body)
        variant = {loop.index.id, *(arg.id for arg in loop.carried_args)}
        moved, kept = [], []
        for op in body:
            if isinstance(op, SSAForRange):
                variant.update(result.id for result in op.results)
                kept.append(op)
                continue
            invariant = (
                op.result is not None and op.opcode in self.MOVABLE and self._safe_anywhere(op)
                and not any(isinstance(x, SSAValue) and x.id in variant for x in op.operands)
            )
            if invariant:
                moved.append(op)
            else:
                if op.result is not None:
                    variant.add(op.result.id)
                kept.append(op)
        return moved, SSAForRange(
            loop.index, loop.start, loop.stop, loop.step, loop.carried_inputs,
            loop.carried_args, kept, loop.yields, loop.results,
        )


def codegen_pipeline(verifier) -> "PassManager":
    """The passes the code generator's input goes through: fold, CSE and DCE inside and
    outside loops, loop-invariant motion, then CSE and DCE once more over what moved."""
    passes = [ConstantFoldPass(), CSEPass(), DCEPass(), LoopInvariantMotionPass(), CSEPass(), DCEPass()]
    return PassManager(passes, verifier, region_aware=True)


class PassManager:
    """Runs passes in order, verifying after each.

    With ``region_aware=False`` (the default, and what produces the SSA handed
    back to callers) a kernel containing a runtime loop is only verified, as in
    the reference.  ``codegen_pipeline`` builds the region-aware manager whose
    output the code generator consumes.
    """

    def __init__(self, passes, verifier, region_aware: bool = False) -> None:
        self.passes = passes
        self.verifier = verifier
        self.region_aware = region_aware

    def run(self, ops):
        if not self.region_aware and any(isinstance(op, SSAForRange) for op in ops):
            self.verifier.verify(ops)
            return ops
        for compiler_pass in self.passes:
            ops = compiler_pass.run(ops)
            self.verifier.verify(ops)
        return ops
