"""Typed SSA: data structures, lowering from the expression tree, text printer.

The value/operation classes, the opcode names, the value numbering (loop index,
then carried arguments, then body, then results) and the printed syntax are the
reference's (``src/mytriton/ssa.py:34-67``, ``:112-352``, ``:383-455``), because
printed SSA is compared literally by existing tests.  The lowering itself is a
table-driven walk: one small method per node class, looked up by class name.
Values created inside a loop body are forgotten when the loop closes, so a
body-local value can never be referenced from outside its region.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from . import nodes as N
from .nodes import Const, Param
from .type_inference import TypeInference
from .types import I32, Type


@dataclass(frozen=True)
class SSAValue:
    id: int
    ty: Type

    def __str__(self) -> str:
        return f"%{self.id}"


SSAOperand = SSAValue | Param | Const | None


@dataclass
class SSAOp:
    opcode: str
    operands: tuple[SSAOperand, ...] = ()
    result: SSAValue | None = None
    attrs: dict[str, object] = field(default_factory=dict)


@dataclass
class SSAForRange:
    index: SSAValue
    start: SSAOperand
    stop: SSAOperand
    step: SSAOperand
    carried_inputs: tuple[SSAOperand, ...]
    carried_args: tuple[SSAValue, ...]
    body: list["SSAItem"]
    yields: tuple[SSAOperand, ...]
    results: tuple[SSAValue, ...]


SSAItem = SSAOp | SSAForRange


class SSALowering:
    BINOPS = {"+": "add", "-": "sub", "*": "mul", "/": "div", "<": "cmp_lt", "&": "and",
              "floordiv": "div", "rem": "rem"}      # on i32 `//` is the same truncating division as `/`

    def __init__(self) -> None:
        self.ops: list[SSAItem] = []
        self.memo: dict[int, SSAOperand] = {}
        self.next_id = 0
        self.type_inference = TypeInference()

    # -- value creation ----------------------------------------------------------

    def new_value(self, ty: Type) -> SSAValue:
        value = SSAValue(self.next_id, ty)
        self.next_id += 1
        return value

    def emit(self, opcode: str, expr: Any, operands=(), attrs=None) -> SSAValue:
        result = self.new_value(self.type_inference.infer(expr))
        self.ops.append(SSAOp(opcode, tuple(operands), result, attrs or {}))
        self.memo[id(expr)] = result
        return result

    # -- expressions -------------------------------------------------------------

    def lower_expr(self, expr: Any) -> SSAOperand:
        if isinstance(expr, (Const, Param)):
            return expr
        seen = self.memo.get(id(expr))
        if seen is not None:
            return seen
        if isinstance(expr, (N.LoopIndex, N.LoopCarry)):
            raise TypeError(f"loop value used outside of loop body: {expr}")
        if isinstance(expr, N.LoopResult):
            raise TypeError("loop result used before loop was lowered")
        handler = getattr(self, "_lower_" + type(expr).__name__, None)
        if handler is None:
            raise TypeError(f"Cannot lower expression: {expr}")
        return handler(expr)

    def _operands(self, *exprs: Any) -> tuple[SSAOperand, ...]:
        return tuple(None if e is None else self.lower_expr(e) for e in exprs)

    def _lower_ProgramId(self, e):
        return self.emit("program_id", e, attrs={"axis": e.axis})

    def _lower_NumPrograms(self, e):
        return self.emit("num_programs", e, attrs={"axis": e.axis})

    def _lower_Arange(self, e):
        return self.emit("arange", e, attrs={"start": e.start, "end": e.end})

    def _lower_Empty(self, e):
        return self.emit("empty", e, attrs={"shape": e.shape, "dtype": e.dtype})

    def _lower_Zeros(self, e):
        return self.emit("zeros", e, attrs={"shape": e.shape, "dtype": e.dtype})

    def _lower_Full(self, e):
        return self.emit(
            "full", e, self._operands(e.value), {"shape": e.shape, "dtype": e.dtype}
        )

    def _lower_BinOp(self, e):
        opcode = self.BINOPS.get(e.op)
        if opcode is None:
            raise TypeError(f"Unsupported binary operator: {e.op}")
        return self.emit(opcode, e, self._operands(e.lhs, e.rhs))

    def _lower_Load(self, e):
        return self.emit("load", e, self._operands(e.ptr, e.mask, e.other))

    def _lower_AddPtr(self, e):
        return self.emit("addptr", e, self._operands(e.base, e.offset))

    def _lower_Maximum(self, e):
        return self.emit("maximum", e, self._operands(e.lhs, e.rhs))

    def _lower_Minimum(self, e):
        return self.emit("minimum", e, self._operands(e.lhs, e.rhs))

    def _lower_UnaryOp(self, e):
        return self.emit(e.op, e, self._operands(e.value))

    def _lower_Where(self, e):
        return self.emit(
            "select", e, self._operands(e.condition, e.true_value, e.false_value)
        )

    def _reduce(self, opcode: str, e):
        # the axis is recorded only for rank-2 operands: rank-1 reductions print as before
        rank2 = getattr(self.type_inference.infer(e.value), "rank", 0) == 2
        return self.emit(opcode, e, self._operands(e.value), {"axis": e.axis} if rank2 else None)

    def _lower_Sum(self, e):
        return self._reduce("sum", e)

    def _lower_Max(self, e):
        return self._reduce("max", e)

    def _lower_Min(self, e):
        return self._reduce("min", e)

    def _lower_ExpandDims(self, e):
        return self.emit("expand_dims", e, self._operands(e.value), {"axis": e.axis})

    def _lower_Dot(self, e):
        attrs = {} if e.input_precision == "ieee" else {"input_precision": e.input_precision}
        return self.emit("dot", e, self._operands(e.lhs, e.rhs, e.acc), attrs)

    # -- statements --------------------------------------------------------------

    def _lower_store(self, store: N.Store) -> None:
        self.type_inference.check_store(store)
        value = self.lower_expr(store.value)
        ptr = self.lower_expr(store.ptr)
        mask = None if store.mask is None else self.lower_expr(store.mask)
        self.ops.append(SSAOp("atomic_add" if store.atomic else "store", (ptr, value, mask)))

    def lower_for_range(self, loop: N.ForRange) -> None:
        outer_ops = self.ops
        snapshot = (dict(self.memo), self.next_id, dict(self.type_inference.types))
        try:
            start, stop, step = self._operands(loop.start, loop.stop, loop.step)
            for captured in loop.captures:
                self.lower_expr(captured)
            carried_inputs = self._operands(*loop.carried_inputs)

            index = self.new_value(I32)
            carried_args = tuple(
                self.new_value(self.type_inference.infer(arg.initial))
                for arg in loop.carried_args
            )

            before_body = dict(self.memo)
            self.memo[id(loop.index)] = index
            for placeholder, arg in zip(loop.carried_args, carried_args, strict=True):
                self.memo[id(placeholder)] = arg

            self.ops = []
            for statement in loop.body:
                self._lower_top_level_op(statement)
            yields = self._operands(*loop.carried_outputs)
            body, self.ops = self.ops, outer_ops

            results = tuple(
                self.new_value(self.type_inference.infer(result)) for result in loop.results
            )
            # leave the region: body-local values and placeholders go out of scope
            self.memo = before_body
            for placeholder, result in zip(loop.results, results, strict=True):
                self.memo[id(placeholder)] = result

            self.ops.append(
                SSAForRange(
                    index, start, stop, step, carried_inputs, carried_args, body, yields, results
                )
            )
        except BaseException:
            self.ops = outer_ops
            self.memo.clear()
            self.memo.update(snapshot[0])
            self.next_id = snapshot[1]
            self.type_inference.types.clear()
            self.type_inference.types.update(snapshot[2])
            raise

    def _lower_top_level_op(self, op: Any) -> None:
        if isinstance(op, N.Store):
            self._lower_store(op)
        elif isinstance(op, N.ForRange):
            self.lower_for_range(op)
        elif isinstance(op, N.BreakUnless):
            self.type_inference.check_break_unless(op)
            self.ops.append(SSAOp("break_unless", (self.lower_expr(op.condition),)))
        else:
            raise TypeError(f"Cannot lower operation: {op}")

    def lower(self, top_level_ops) -> list[SSAItem]:
        for op in top_level_ops:
            self._lower_top_level_op(op)
        return self.ops


class SSAPrinter:
    def operand(self, value: SSAOperand) -> str:
        if value is None:
            return "none"
        if isinstance(value, SSAValue):
            return str(value)
        if isinstance(value, Param):
            return value.name
        if isinstance(value, Const):
            return repr(value.value)
        raise TypeError(f"Unknown SSA operand: {value}")

    def print_op(self, op: SSAOp) -> str:
        text = op.opcode
        if op.operands:
            text += " " + ", ".join(map(self.operand, op.operands))
        if op.attrs:
            text += " {" + ", ".join(f"{k}={v}" for k, v in op.attrs.items()) + "}"
        if op.result is None:
            return text
        return f"{op.result} = {text} : {op.result.ty}"

    def print_for_range(self, loop: SSAForRange) -> list[str]:
        head = ""
        if loop.results:
            head = ", ".join(map(str, loop.results)) + " = "
        head += (
            f"for {loop.index} in range({self.operand(loop.start)}, "
            f"{self.operand(loop.stop)}, {self.operand(loop.step)})"
        )
        if loop.carried_args:
            pairs = zip(loop.carried_args, loop.carried_inputs, strict=True)
            head += " iter_args(" + ", ".join(
                f"{arg} = {self.operand(initial)}" for arg, initial in pairs
            ) + ")"
        if loop.results:
            head += " : " + ", ".join(str(result.ty) for result in loop.results)
        lines = [head + " {"]
        lines += ["  " + line for line in self._lines(loop.body)]
        tail = ", ".join(map(self.operand, loop.yields))
        lines.append(f"  yield {tail}" if tail else "  yield")
        lines.append("}")
        return lines

    def _lines(self, ops) -> list[str]:
        out: list[str] = []
        for op in ops:
            if isinstance(op, SSAForRange):
                out += self.print_for_range(op)
            else:
                out.append(self.print_op(op))
        return out

    def print_ops(self, ops: list[SSAItem]) -> str:
        return "\n".join(self._lines(ops))
