"""AST frontend: run a kernel's Python source symbolically and record its ops.

``trace(fn, signature, bound_args)`` parses the function with ``ast`` and walks
it with a small interpreter whose environment maps names to Python constants
(constexpr parameters, closure/global names) or to symbolic ``Value``/``Ptr``
objects.  ``tl.*`` calls are really executed and grow the expression tree;
``tl.store`` and runtime loops append to the active ``Builder``.

Behaviour and diagnostics mirror the reference's ``src/mytriton/ast_frontend.py``:
loops over Python ints are unrolled (``:214-243``); other loops become one
``ForRange`` whose carried values are the pre-existing names assigned in the
body, in first-assignment order, and whose ``captures`` are the outer symbolic
values read in the body (``:245-331``).  The implementation is a dispatch-table
interpreter (``_stmt_*`` / ``_expr_*`` methods keyed by AST class name) rather
than an ``ast.NodeVisitor``.
"""

from __future__ import annotations

import ast
import inspect
import textwrap
from collections.abc import Mapping
from typing import Any

from . import language as tl
from . import trace as trace_state
from .nodes import BinOp, BreakUnless, ForRange, LoopCarry, LoopIndex, LoopResult, UnaryOp
from .trace import Builder, Ptr, Value, is_constexpr_annotation, make_runtime_params, unwrap
from .type_inference import TypeInference
from .types import BOOL, I32, PointerType, element_of


class ASTFrontendError(TypeError):
    pass


class _Unbound:
    """Environment marker: the name is assigned on only one path of a run-time ``if``."""

    def __init__(self, name: str) -> None:
        self.name = name


def _function_def(fn) -> ast.FunctionDef:
    module = ast.parse(textwrap.dedent(inspect.getsource(fn)))
    for node in module.body:
        if isinstance(node, ast.FunctionDef) and node.name == fn.__name__:
            return node
    raise ASTFrontendError(f"could not find function definition for {fn.__name__}")


def _initial_env(signature, bound_args: Mapping[str, Any], runtime_params) -> dict[str, Any]:
    by_name = {param.name: param for param in runtime_params}
    env: dict[str, Any] = {}
    for name, parameter in signature.parameters.items():
        if is_constexpr_annotation(parameter.annotation):
            env[name] = bound_args[name]
        else:
            param = by_name[name]
            env[name] = Ptr(param) if isinstance(param.ty, PointerType) else Value(param)
    return env


_ASSIGN_KIND = {
    ast.Assign: "assignment",
    ast.AnnAssign: "annotated assignment",
    ast.AugAssign: "augmented assignment",
}


def _assigned_names(body: list[ast.stmt]) -> list[str]:
    """Names bound by assignment statements anywhere under ``body``, source order."""
    names: dict[str, None] = {}

    def scan(node: ast.AST) -> None:
        kind = _ASSIGN_KIND.get(type(node))
        if kind is not None:
            targets = node.targets if isinstance(node, ast.Assign) else [node.target]
            for target in targets:
                if not isinstance(target, ast.Name):
                    raise ASTFrontendError(f"loop MVP supports only {kind} to simple names")
                names.setdefault(target.id)
            if node.value is not None:
                scan(node.value)
            return
        for child in ast.iter_child_nodes(node):
            scan(child)

    for statement in body:
        scan(statement)
    return list(names)


def _has_jump(body: list[ast.stmt]) -> bool:
    """Whether ``break`` or ``continue`` of *this* loop occurs under ``body`` (nested loops own theirs)."""
    for statement in body:
        if isinstance(statement, (ast.Break, ast.Continue)):
            return True
        if isinstance(statement, ast.If) and (_has_jump(statement.body) or _has_jump(statement.orelse)):
            return True
    return False


def _assign_flag(name: str, value: bool, like: ast.AST) -> ast.stmt:
    return ast.copy_location(ast.Assign(
        targets=[ast.Name(id=name, ctx=ast.Store())], value=ast.Constant(value=value), lineno=0), like)


def _rewrite_jumps(body: list[ast.stmt], skip: str, stop: str) -> tuple[list[ast.stmt], bool]:
    """``break`` and ``continue`` of one loop body as flags and ``if`` statements, which the tracer
    already lowers (by predication when the condition is a run-time value):

    * ``continue`` becomes ``skip = True``, ``break`` becomes ``stop = True; skip = True``; what
      follows either in the same block is dead;
    * the statements after an ``if`` that may have jumped run under ``if not skip:``.

    The caller resets ``skip`` at the top of the body and, for ``break``, carries ``stop``
    through the loop and leaves the loop when it is set.  Returns (statements, uses ``break``)."""
    uses_break = False

    def rewrite(statements: list[ast.stmt]) -> tuple[list[ast.stmt], bool]:
        nonlocal uses_break
        out: list[ast.stmt] = []
        for position, statement in enumerate(statements):
            if isinstance(statement, ast.Continue):
                out.append(_assign_flag(skip, True, statement))
                return out, True
            if isinstance(statement, ast.Break):
                uses_break = True
                out.extend([_assign_flag(stop, True, statement), _assign_flag(skip, True, statement)])
                return out, True
            if isinstance(statement, ast.If) and (_has_jump(statement.body) or _has_jump(statement.orelse)):
                then, _ = rewrite(statement.body)
                otherwise, _ = rewrite(statement.orelse)
                out.append(ast.copy_location(
                    ast.If(test=statement.test, body=then or [ast.Pass()], orelse=otherwise), statement))
                rest, _ = rewrite(statements[position + 1:])
                if rest:
                    guard = ast.UnaryOp(op=ast.Not(), operand=ast.Name(id=skip, ctx=ast.Load()))
                    out.append(ast.fix_missing_locations(ast.copy_location(
                        ast.If(test=guard, body=rest, orelse=[]), statement)))
                return out, True
            out.append(statement)
        return out, False

    statements, jumped = rewrite(body)
    if jumped:
        statements = [_assign_flag(skip, False, body[0])] + statements
    return [ast.fix_missing_locations(statement) for statement in statements], uses_break


_BINARY = {
    ast.Add: lambda a, b: a + b,
    ast.Sub: lambda a, b: a - b,
    ast.Mult: lambda a, b: a * b,
    ast.Div: lambda a, b: a / b,
    ast.FloorDiv: lambda a, b: a // b,
    ast.Mod: lambda a, b: a % b,
    ast.BitAnd: lambda a, b: a & b,
}
_AUGMENTED = {key: _BINARY[key] for key in (ast.Add, ast.Sub, ast.Mult, ast.Div)}
_PYTHON_COMPARE = {
    ast.Eq: lambda a, b: a == b, ast.NotEq: lambda a, b: a != b, ast.Gt: lambda a, b: a > b,
    ast.GtE: lambda a, b: a >= b, ast.LtE: lambda a, b: a <= b, ast.IsNot: lambda a, b: a is not b,
}


class ASTTracer:
    """Symbolic interpreter for one statement list (the kernel or a loop body)."""

    def __init__(
        self,
        env: dict[str, Any],
        external_env: Mapping[str, Any],
        capture_env: Mapping[str, Any] | None = None,
    ) -> None:
        self.env = env
        self.external_env = external_env
        self.captures: list[Any] = []
        self.in_runtime_loop = False
        self._returned = False          # a return was traced in the statement list being visited
        self.inlined = False            # tracing the body of a @jit helper called from a kernel
        self.return_value: Any = None
        self._capturable = {
            id(unwrap(value))
            for value in (capture_env or {}).values()
            if isinstance(value, (Ptr, Value))
        }

    # -- capture bookkeeping -----------------------------------------------------

    def _note_capture(self, expr: Any) -> None:
        if id(expr) in self._capturable:
            self._capturable.discard(id(expr))
            self.captures.append(expr)

    # -- dispatch ----------------------------------------------------------------

    def visit_stmt_list(self, body: list[ast.stmt]) -> None:
        for statement in body:
            if self._returned:
                break                   # statements after a return are dead
            self.visit(statement)

    def visit(self, node: ast.AST) -> Any:
        kind = type(node).__name__
        handler = getattr(self, "_stmt_" + kind, None) or getattr(self, "_expr_" + kind, None)
        if handler is None:
            raise ASTFrontendError(f"unsupported AST node: {kind}")
        return handler(node)

    # -- statements --------------------------------------------------------------

    def _stmt_Expr(self, node: ast.Expr) -> None:
        self.visit(node.value)

    def _stmt_Return(self, node: ast.Return) -> None:
        """A bare ``return`` ends the program: what follows it in the same block is not
        traced, and when it sits under a run-time ``if`` every later load and store is
        masked by the negated condition.  Kernels return nothing, so a value is refused."""
        if self.inlined:
            # a helper returns a value to the kernel that called it; the helper's own
            # statements after the return are not traced
            if trace_state.branch_predicate() is not self.entry_predicate:
                raise ASTFrontendError("a helper may not return from inside a run-time if")
            if self.in_runtime_loop is not self.entry_in_loop:
                raise ASTFrontendError("a helper may not return from inside a runtime loop")
            self.return_value = None if node.value is None else self.visit(node.value)
            self._returned = True
            return
        if node.value is not None:
            raise ASTFrontendError("return statements are not supported in kernels")
        if self.in_runtime_loop:
            raise ASTFrontendError("return inside a runtime loop is not supported")
        branch = trace_state.branch_predicate()
        if branch is not None:
            trace_state.add_exit(UnaryOp("not", branch))
        self._returned = True

    def _stmt_Assign(self, node: ast.Assign) -> None:
        if len(node.targets) != 1:
            raise ASTFrontendError("only single-target assignment is supported")
        (target,) = node.targets
        if not isinstance(target, ast.Name):
            raise ASTFrontendError("only assignment to a simple name is supported")
        self.env[target.id] = self.visit(node.value)

    def _stmt_AnnAssign(self, node: ast.AnnAssign) -> None:
        if not isinstance(node.target, ast.Name):
            raise ASTFrontendError("only assignment to a simple name is supported")
        self.env[node.target.id] = None if node.value is None else self.visit(node.value)

    def _stmt_AugAssign(self, node: ast.AugAssign) -> None:
        if not isinstance(node.target, ast.Name):
            raise ASTFrontendError("only augmented assignment to a simple name is supported")
        name = node.target.id
        if name not in self.env:
            raise NameError(name)
        current = self.env[name]
        update = self.visit(node.value)
        combine = _AUGMENTED.get(type(node.op))
        if combine is None:
            raise ASTFrontendError(
                f"unsupported augmented assignment: {type(node.op).__name__}"
            )
        self.env[name] = combine(current, update)

    def _stmt_If(self, node: ast.If) -> None:
        """``if`` on a compile-time condition (constexpr parameters, Python values) picks
        a branch while tracing.  The reference rejects every ``if`` statement; conditions
        on symbolic values are still refused here (use ``tl.where``)."""
        test = self.visit(node.test)
        if isinstance(test, Ptr):
            raise ASTFrontendError("a pointer is not a condition")
        if isinstance(test, Value):
            self._runtime_if(node, test)
        else:
            self.visit_stmt_list(node.body if test else node.orelse)

    def _runtime_if(self, node: ast.If, test: Value) -> None:
        """``if`` on a run-time scalar, by predication: both branches are traced, their
        loads and stores masked by the branch condition, and every name the branches leave
        with different values becomes ``where(condition, then value, else value)``."""
        condition = unwrap(test)
        try:
            condition_type = TypeInference().infer(condition)
        except TypeError as error:
            raise ASTFrontendError(f"cannot type the if condition: {error}") from error
        if condition_type != BOOL:
            raise ASTFrontendError(
                f"an if condition must be a scalar boolean, got {condition_type}; "
                "use tl.where for data-dependent selection on blocks"
            )
        outer = trace_state.branch_predicate()
        within = (lambda expr: expr) if outer is None else (lambda expr: BinOp("&", outer, expr))
        before = dict(self.env)

        def run(body: list[ast.stmt], predicate: Any) -> dict[str, Any]:
            self.env.clear()
            self.env.update(before)
            with trace_state.predicated(within(predicate)):
                self.visit_stmt_list(body)
            self._returned = False      # a return inside the branch ends only that branch's trace
            return dict(self.env)

        then_env = run(node.body, condition)
        else_env = run(node.orelse, UnaryOp("not", condition)) if node.orelse else before
        merged: dict[str, Any] = {}
        for name in list(then_env) + [name for name in else_env if name not in then_env]:
            if name in then_env and name in else_env:
                merged[name] = self._merge(name, test, then_env[name], else_env[name])
            else:
                merged[name] = _Unbound(name)       # defined on one path only
        self.env.clear()
        self.env.update(merged)

    @staticmethod
    def _merge(name: str, test: Value, taken: Any, skipped: Any) -> Any:
        if taken is skipped:
            return taken
        if isinstance(taken, _Unbound) or isinstance(skipped, _Unbound):
            return _Unbound(name)
        if isinstance(taken, Ptr) or isinstance(skipped, Ptr):
            raise ASTFrontendError(f"pointer {name!r} may not depend on a run-time condition")
        symbolic = isinstance(taken, Value) or isinstance(skipped, Value)
        if not symbolic:
            if type(taken) is type(skipped) and taken == skipped:
                return taken
            if not all(isinstance(value, (bool, int, float)) for value in (taken, skipped)):
                raise ASTFrontendError(
                    f"{name!r} is bound to different compile-time objects on the two paths of a run-time if"
                )
        if ASTTracer._is_boolean(taken) and ASTTracer._is_boolean(skipped):
            return ASTTracer._merge_booleans(test, taken, skipped)
        return tl.where(test, taken, skipped)

    @staticmethod
    def _is_boolean(value: Any) -> bool:
        if isinstance(value, bool):
            return True
        if not isinstance(value, Value):
            return False
        try:
            return TypeInference().infer(unwrap(value)) == BOOL
        except TypeError:
            return False

    @staticmethod
    def _merge_booleans(test: Value, taken: Any, skipped: Any) -> Any:
        """(test and taken) or (not test and skipped) with the operators booleans have here, `&` and
        `not` (a flag set on one path of a run-time if: there is no select of booleans)."""
        def both(a: Any, b: Any) -> Any:        # a & b with compile-time operands folded
            if isinstance(a, bool):
                return b if a else False
            if isinstance(b, bool):
                return a if b else False
            return a & b

        def negate(a: Any) -> Any:
            return (not a) if isinstance(a, bool) else ~a

        on_taken, on_skipped = both(test, taken), both(negate(test), skipped)
        return negate(both(negate(on_taken), negate(on_skipped)))

    def _stmt_Pass(self, node: ast.Pass) -> None:
        return None

    def _stmt_For(self, node: ast.For) -> None:
        if not isinstance(node.target, ast.Name):
            raise ASTFrontendError(
                "only for loops with a simple induction variable are supported"
            )
        if node.orelse:
            raise ASTFrontendError("for/else is not supported")
        start, stop, step = self._range_bounds(node.iter)
        if all(type(bound) is int for bound in (start, stop, step)):
            self._unroll(node, range(start, stop, step))
        else:
            self._runtime_loop(node, start, stop, step)

    _jump_flags = 0         # loops rewritten so far: their flag names must not collide

    @classmethod
    def _flag_names(cls) -> tuple[str, str]:
        cls._jump_flags += 1
        return f"_mtb_skip_{cls._jump_flags}", f"_mtb_stop_{cls._jump_flags}"

    def _unroll(self, node: ast.For, trip: range) -> None:
        name = node.target.id
        missing = object()
        saved = self.env.get(name, missing)
        body = node.body
        if _has_jump(body):
            # the iterations are traced one after the other: after a break the remaining ones are
            # skipped while tracing (a compile-time condition) or predicated (a run-time one)
            skip, stop = self._flag_names()
            body, _ = _rewrite_jumps(body, skip, stop)
            self.env[stop] = False
            guard = ast.UnaryOp(op=ast.Not(), operand=ast.Name(id=stop, ctx=ast.Load()))
            body = [ast.fix_missing_locations(ast.copy_location(ast.If(test=guard, body=body, orelse=[]), node))]
        for value in trip:
            self.env[name] = value
            self.visit_stmt_list(body)
        if saved is missing:
            self.env.pop(name, None)
        else:
            self.env[name] = saved

    def _stmt_While(self, node: ast.While) -> None:
        """``while`` on a run-time scalar condition: a counted loop with the largest i32
        bound whose body starts by testing the condition and leaving the loop when it is
        false (``BreakUnless``).  Carried names follow the ``for`` rule.  Inside a run-time
        ``if`` the branch condition is part of the test, so a loop in a branch that is not
        taken ends at once."""
        if node.orelse:
            raise ASTFrontendError("while/else is not supported")
        self._region_loop(node.body, None, 0, 2**31 - 1, 1, test=node.test)

    def _runtime_loop(self, node: ast.For, start: Any, stop: Any, step: Any) -> None:
        if type(step) is not int:
            raise ASTFrontendError("runtime for MVP requires integer constant step")
        if step <= 0:
            raise ASTFrontendError("runtime for MVP supports only positive step")
        self._region_loop(node.body, node.target.id, start, stop, step)

    def _region_loop(self, body: list[ast.stmt], induction: str | None, start: Any, stop: Any,
                     step: Any, test: ast.expr | None = None) -> None:
        leave: ast.expr | None = None
        if _has_jump(body):
            # `continue` skips the rest of the body under a flag; `break` also sets a flag that is
            # carried through the loop, and the body starts by leaving the loop when it is set
            skip_flag, stop_flag = self._flag_names()
            body, uses_break = _rewrite_jumps(body, skip_flag, stop_flag)
            if uses_break:
                self.env[stop_flag] = False
                leave = ast.fix_missing_locations(ast.copy_location(
                    ast.UnaryOp(op=ast.Not(), operand=ast.Name(id=stop_flag, ctx=ast.Load())), body[0]))
        assigned = _assigned_names(body)
        if induction in assigned:
            raise ASTFrontendError(
                "assignment to runtime loop induction variable is not supported"
            )

        # names that exist before the loop and are rebound inside it are carried
        carried = [name for name in assigned
                   if name in self.env and not isinstance(self.env[name], _Unbound)]
        inputs = tuple(unwrap(self.env[name]) for name in carried)
        placeholders = tuple(LoopCarry(index=i, initial=init) for i, init in enumerate(inputs))
        index = LoopIndex(induction if induction is not None else "while")

        body_env = dict(self.env)
        if induction is not None:
            body_env[induction] = Value(index)
        # a carried pointer (``ptrs += BLOCK`` in the body) stays a pointer inside and after the loop
        wrappers = [Ptr if isinstance(self.env[name], Ptr) else Value for name in carried]
        body_env.update({name: wrap(ph) for name, wrap, ph in zip(carried, wrappers, placeholders)})
        visible = {
            name: value
            for name, value in self.env.items()
            if name != induction and name not in carried
        }

        with Builder() as body_builder:
            inner = ASTTracer(body_env, self.external_env, capture_env=visible)
            inner.in_runtime_loop = True
            forever = isinstance(test, ast.Constant) and test.value is True and leave is not None
            if test is not None and not forever:        # `while True:` with a break has no test of its own
                body_builder.ops.append(BreakUnless(inner._loop_condition(test)))
            if leave is not None:
                body_builder.ops.append(BreakUnless(inner._loop_condition(leave)))
            inner.visit_stmt_list(body)
        for captured in inner.captures:
            self._note_capture(captured)

        loop = ForRange(
            index=index,
            start=unwrap(start),
            stop=unwrap(stop),
            step=unwrap(step),
            captures=tuple(inner.captures) + self._predicate_captures(),
            body=body_builder.ops,
            carried_inputs=inputs,
            carried_args=placeholders,
            carried_outputs=tuple(unwrap(body_env[name]) for name in carried),
        )
        loop.results = tuple(LoopResult(loop=loop, index=i) for i in range(len(carried)))
        Builder.current().ops.append(loop)
        for name, wrap, result in zip(carried, wrappers, loop.results):
            self.env[name] = wrap(result)

    def _loop_condition(self, test: ast.expr) -> Any:
        value = self.visit(test)
        if not isinstance(value, Value):
            raise ASTFrontendError(
                "a while condition must depend on run-time values (or be True, with a break in the body)"
            )
        condition = unwrap(value)
        try:
            condition_type = TypeInference().infer(condition)
        except TypeError as error:
            raise ASTFrontendError(f"cannot type the while condition: {error}") from error
        if condition_type != BOOL:
            raise ASTFrontendError(f"a while condition must be a scalar boolean, got {condition_type}")
        predicate = trace_state.active_predicate()
        return condition if predicate is None else BinOp("&", condition, predicate)

    @staticmethod
    def _predicate_captures() -> tuple[Any, ...]:
        """The predicate in force is read by every masked access of a loop body, so it is
        lowered ahead of the loop like any other outer value the body uses."""
        predicate = trace_state.active_predicate()
        return () if predicate is None else (predicate,)

    # -- expressions -------------------------------------------------------------

    def _expr_Name(self, node: ast.Name) -> Any:
        if isinstance(node.ctx, ast.Store):
            return node.id
        if not isinstance(node.ctx, ast.Load):
            raise ASTFrontendError(f"unsupported name context: {type(node.ctx).__name__}")
        if node.id in self.env:
            value = self.env[node.id]
            if isinstance(value, _Unbound):
                raise ASTFrontendError(
                    f"{node.id!r} is assigned on only one path of a run-time if and used after it"
                )
            if isinstance(value, (Ptr, Value)):
                self._note_capture(unwrap(value))
            return value
        if node.id in self.external_env:
            return self.external_env[node.id]
        raise NameError(node.id)

    def _expr_Constant(self, node: ast.Constant) -> Any:
        return node.value

    def _expr_Tuple(self, node: ast.Tuple) -> tuple[Any, ...]:
        return tuple(self.visit(item) for item in node.elts)

    def _expr_List(self, node: ast.List) -> list[Any]:
        return [self.visit(item) for item in node.elts]

    def _expr_Attribute(self, node: ast.Attribute) -> Any:
        return getattr(self.visit(node.value), node.attr)

    def _expr_Call(self, node: ast.Call) -> Any:
        callee = self.visit(node.func)
        positional = [self.visit(argument) for argument in node.args]
        named = {}
        for keyword in node.keywords:
            if keyword.arg is None:
                raise ASTFrontendError("**kwargs are not supported")
            named[keyword.arg] = self.visit(keyword.value)
        if type(callee).__name__ == "CompiledKernel" and hasattr(callee, "fn"):
            return self._inline(callee, positional, named)
        return callee(*positional, **named)

    def _inline(self, helper: Any, positional: list[Any], named: dict[str, Any]) -> Any:
        """A ``@triton.jit`` function called from a kernel is traced in place: its parameters
        are bound to the argument values (symbolic or compile-time), its statements append
        to the same builder, and the value of its ``return`` is the value of the call."""
        try:
            bound = helper.signature.bind(*positional, **named)
        except TypeError as error:
            raise ASTFrontendError(f"{helper.fn.__name__}(): {error}") from error
        bound.apply_defaults()
        scope = inspect.getclosurevars(helper.fn)
        external = {**scope.builtins, **scope.globals, **scope.nonlocals}
        inner = ASTTracer(dict(bound.arguments), external)
        inner.inlined = True
        inner.in_runtime_loop = inner.entry_in_loop = self.in_runtime_loop
        inner.entry_predicate = trace_state.branch_predicate()
        inner.visit_stmt_list(_function_def(helper.fn).body)
        return inner.return_value

    def _expr_BinOp(self, node: ast.BinOp) -> Any:
        lhs, rhs = self.visit(node.left), self.visit(node.right)
        combine = _BINARY.get(type(node.op))
        if combine is None:
            raise ASTFrontendError(f"unsupported binary operator: {type(node.op).__name__}")
        return combine(lhs, rhs)

    def _expr_UnaryOp(self, node: ast.UnaryOp) -> Any:
        operand = self.visit(node.operand)
        if isinstance(node.op, ast.USub):
            return -operand
        if isinstance(node.op, ast.UAdd):
            return operand
        if isinstance(node.op, (ast.Not, ast.Invert)) and isinstance(operand, Value):
            return ~operand                   # boolean negation (type-checked later)
        if isinstance(node.op, ast.Not) and not isinstance(operand, Ptr):
            return not operand
        raise ASTFrontendError(f"unsupported unary operator: {type(node.op).__name__}")

    def _expr_Compare(self, node: ast.Compare) -> Any:
        if len(node.ops) != 1:
            raise ASTFrontendError(
                "only simple comparisons are supported; "
                "when combining comparisons with &, wrap each comparison in parentheses"
            )
        lhs, rhs = self.visit(node.left), self.visit(node.comparators[0])
        if isinstance(node.ops[0], ast.Lt):
            return lhs < rhs
        if isinstance(node.ops[0], ast.Gt) and (isinstance(lhs, Value) or isinstance(rhs, Value)):
            return lhs > rhs                  # lowered as rhs < lhs
        if isinstance(node.ops[0], ast.GtE) and (isinstance(lhs, Value) or isinstance(rhs, Value)):
            return ~(lhs < rhs)               # a >= b is not (a < b)
        if isinstance(node.ops[0], ast.LtE) and (isinstance(lhs, Value) or isinstance(rhs, Value)):
            return ~(lhs > rhs)               # a <= b is not (b < a)
        if isinstance(node.ops[0], (ast.Eq, ast.NotEq)) and (isinstance(lhs, Value) or isinstance(rhs, Value)):
            # integers only: neither is smaller.  (For floats that would call NaN equal to itself.)
            if not (self._is_integer(lhs) and self._is_integer(rhs)):
                raise ASTFrontendError(
                    "== and != on run-time values are supported for integers only; "
                    "compare floating-point values with < and >")
            same = ~(lhs < rhs) & ~(lhs > rhs)
            return same if isinstance(node.ops[0], ast.Eq) else ~same
        if isinstance(node.ops[0], ast.Is):
            return lhs is rhs
        compare = _PYTHON_COMPARE.get(type(node.ops[0]))
        if compare is not None and not isinstance(lhs, (Value, Ptr)) and not isinstance(rhs, (Value, Ptr)):
            return compare(lhs, rhs)          # compile-time values: any Python comparison
        raise ASTFrontendError(
            f"unsupported comparison operator: {type(node.ops[0]).__name__}"
        )

    @staticmethod
    def _is_integer(value: Any) -> bool:
        if isinstance(value, bool):
            return False
        if isinstance(value, int):
            return True
        if not isinstance(value, Value):
            return False
        try:
            return element_of(TypeInference().infer(unwrap(value))) == I32
        except TypeError:
            return False

    def _expr_Subscript(self, node: ast.Subscript) -> Any:
        return self.visit(node.value)[self._index(node.slice)]

    def _expr_IfExp(self, node: ast.IfExp) -> Any:
        test = self.visit(node.test)
        if not isinstance(test, bool):
            raise ASTFrontendError("only constexpr conditions in IfExp are supported")
        return self.visit(node.body if test else node.orelse)

    # -- helpers -----------------------------------------------------------------

    def _index(self, node: ast.AST) -> Any:
        if isinstance(node, ast.Tuple):
            return tuple(self._index(item) for item in node.elts)
        if isinstance(node, ast.Slice):
            if node.lower is node.upper is node.step is None:
                return slice(None)
            raise ASTFrontendError("only ':' slices are supported")
        if isinstance(node, ast.Constant) and node.value is None:
            return None
        return self.visit(node)

    def _range_bounds(self, node: ast.AST) -> tuple[Any, Any, Any]:
        if not isinstance(node, ast.Call):
            raise ASTFrontendError("only for ... in range(...) is supported")
        iterator = self.visit(node.func)
        bounds = [self.visit(argument) for argument in node.args]
        if iterator is not range and iterator is not tl.static_range:
            raise ASTFrontendError(
                "only range(...) and tl.static_range(...) loops are supported"
            )
        if len(bounds) == 1:
            return 0, bounds[0], 1
        if len(bounds) == 2:
            return bounds[0], bounds[1], 1
        if len(bounds) == 3:
            return bounds[0], bounds[1], bounds[2]
        raise ASTFrontendError("range expects 1, 2, or 3 arguments")


def trace(fn, signature, bound_args, runtime_params=None, constants=None):
    """Trace ``fn`` into ``(top_level_ops, runtime_params)``.  ``constants`` names run-time scalar
    arguments whose value is folded into the IR (they stay in the parameter list)."""
    if runtime_params is None:
        runtime_params = make_runtime_params(signature, bound_args)
    definition = _function_def(fn)
    env = _initial_env(signature, bound_args, runtime_params)
    env.update(constants or {})
    scope = inspect.getclosurevars(fn)
    external = {**scope.builtins, **scope.globals, **scope.nonlocals}
    with Builder() as builder, trace_state.guards_reset():
        ASTTracer(env, external).visit_stmt_list(definition.body)
    return builder.ops, runtime_params
