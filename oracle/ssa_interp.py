"""NumPy interpreter of printed typed-SSA — TEST INFRASTRUCTURE, not product code.

``run(ssa_text, args, grid)`` executes a kernel, one program id at a time, on the
host.  It parses the SSA *text* (the form ``SSAPrinter`` prints, which the golden
fixtures pin to the reference's own output), so it shares no code with the
package under test.

Per-opcode meaning follows what the reference's code generator emits for one
thread (``src/mytriton/cuda_codegen.py``), evaluated for all elements of a block
at once:

* arithmetic is C arithmetic on ``int``/``float``: i32 ``/`` truncates toward
  zero (``:37-44``), mixed i32/f32 promotes to f32;
* ``maximum``/``minimum`` on f32 propagate NaN and return the right operand on
  ties, ``isnan(l) ? l : (isnan(r) ? r : (l > r ? l : r))`` (``:366-376``);
* ``load`` is ``mask ? base[idx] : other`` with ``other`` defaulting to zero and
  masked-off addresses never touched (``:349-365``); ``store`` is
  ``if (mask) base[idx] = value`` (``:282-300``);
* ``sum``/``max``/``min`` run the same shared-memory tree, stride = W/2 .. 1,
  ``a[t] op= a[t+stride]`` with ``fmaxf``/``fminf`` for f32 (``:155-232``), so
  the fp32 summation order is the reference's;
* ``for`` carries values exactly as ``emit_for_range`` does (``:234-279``).

``dot`` (absent from the reference) is evaluated in float64 and rounded once.
"""

from __future__ import annotations

import ast
import itertools
import re
from dataclasses import dataclass
from typing import Any

import numpy as np

_INT = np.int32
_F32 = np.float32


@dataclass
class _Ptr:
    base: str
    index: Any  # int32 scalar or array


@dataclass
class _Op:
    results: list[int]
    opcode: str
    operands: list[str]
    attrs: dict[str, Any]
    ty: str | None


# f32 -> f32 opcodes beyond exp, with NumPy's float32 functions as their meaning
_FLOAT_UNARY = {
    "sqrt": np.sqrt, "rsqrt": lambda x: np.float32(1.0) / np.sqrt(x), "log": np.log, "log2": np.log2,
    "exp2": np.exp2, "sin": np.sin, "cos": np.cos, "tanh": np.tanh, "abs": np.abs,
    "round_f16": lambda x: np.asarray(x, np.float32).astype(np.float16).astype(np.float32),
    "round_bf16": lambda x: _round_to_bf16(np.asarray(x, np.float32)),
}


def _round_to_bf16(x: np.ndarray) -> np.ndarray:
    """fp32 -> nearest bf16 (ties to even) -> fp32, NaN kept."""
    bits = x.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return np.where(np.isnan(x), x, rounded.view(np.float32))


class _LeaveLoop(Exception):
    """Raised by ``break_unless`` with a false condition; caught by the innermost loop."""


@dataclass
class _Loop:
    results: list[int]
    index: int
    bounds: list[str]
    carried: list[tuple[int, str]]
    body: list[Any]
    yields: list[str]


_TYPE_RE = re.compile(r"^(?:vector<(\d+) x (.+)>|block<([\dx]+) x (.+)>|(.+))$")


def _parse_type(text: str) -> tuple[tuple[int, ...], str]:
    m = _TYPE_RE.match(text.strip())
    if m.group(1):
        return (int(m.group(1)),), m.group(2)
    if m.group(3):
        return tuple(int(d) for d in m.group(3).split("x")), m.group(4)
    return (), m.group(5)


def _split_operands(text: str) -> list[str]:
    return [part.strip() for part in text.split(",")] if text.strip() else []


def _parse_attrs(text: str) -> dict[str, Any]:
    attrs: dict[str, Any] = {}
    # key=value pairs; values may contain commas inside parentheses
    depth, start, parts = 0, 0, []
    for i, ch in enumerate(text):
        depth += ch in "(["
        depth -= ch in ")]"
        if ch == "," and depth == 0:
            parts.append(text[start:i])
            start = i + 1
    parts.append(text[start:])
    for part in parts:
        key, _, value = part.strip().partition("=")
        try:
            attrs[key] = ast.literal_eval(value)
        except (ValueError, SyntaxError):
            attrs[key] = value
    return attrs


def _parse_block(lines: list[str], pos: int, indent: int) -> tuple[list[Any], list[str], int]:
    """Parse statements at ``indent`` until a `yield`/`}`; returns (ops, yields, next_pos)."""
    ops: list[Any] = []
    yields: list[str] = []
    pad = " " * indent
    while pos < len(lines):
        raw = lines[pos]
        line = raw[indent:] if raw.startswith(pad) else raw.strip()
        if line.startswith("yield"):
            yields = _split_operands(line[5:])
            return ops, yields, pos + 1
        if line == "}":
            return ops, yields, pos
        loop = re.match(
            r"^(?:((?:%\d+)(?:, %\d+)*) = )?for %(\d+) in range\((.*?)\)"
            r"(?: iter_args\((.*?)\))?(?: : .*)? \{$",
            line,
        )
        if loop:
            results = [int(x[1:]) for x in _split_operands(loop.group(1) or "")]
            carried = []
            for pair in _split_operands(loop.group(4) or ""):
                arg, _, init = pair.partition(" = ")
                carried.append((int(arg.strip()[1:]), init.strip()))
            body, body_yields, pos = _parse_block(lines, pos + 1, indent + 2)
            assert lines[pos].strip() == "}"
            ops.append(_Loop(results, int(loop.group(2)), _split_operands(loop.group(3)),
                             carried, body, body_yields))
            pos += 1
            continue
        m = re.match(r"^(?:%(\d+) = )?(.*)$", line)
        results = [int(m.group(1))] if m.group(1) else []
        rest, ty = m.group(2), None
        if results:
            rest, _, ty = rest.rpartition(" : ")
        attrs: dict[str, Any] = {}
        brace = re.search(r" \{(.*)\}$", rest)
        if brace:
            attrs = _parse_attrs(brace.group(1))
            rest = rest[: brace.start()]
        opcode, _, operand_text = rest.partition(" ")
        ops.append(_Op(results, opcode, _split_operands(operand_text), attrs, ty))
        pos += 1
    return ops, yields, pos


def parse(ssa_text: str) -> list[Any]:
    ops, _, _ = _parse_block(ssa_text.splitlines(), 0, 0)
    return ops


# ----------------------------------------------------------------------------- evaluation


def _tree_reduce(values: np.ndarray, opcode: str) -> Any:
    work = values.copy()
    stride = work.shape[0] // 2
    while stride > 0:
        lhs, rhs = work[:stride], work[stride: 2 * stride]
        if opcode == "sum":
            work[:stride] = lhs + rhs
        elif work.dtype == _F32:
            work[:stride] = np.fmax(lhs, rhs) if opcode == "max" else np.fmin(lhs, rhs)
        else:
            work[:stride] = np.maximum(lhs, rhs) if opcode == "max" else np.minimum(lhs, rhs)
        stride //= 2
    return work[0]


def _axis_reduce(values: np.ndarray, opcode: str, axis: int) -> np.ndarray:
    """Reduction of a rank-2 block along ``axis``.  Sums are taken in float64 (the device's
    order of additions is an implementation matter; comparisons use a tolerance); extrema
    ignore NaNs the way fmaxf / fminf do."""
    if opcode == "sum":
        wide = values.astype(np.float64 if values.dtype == _F32 else np.int64)
        return wide.sum(axis=axis)
    if values.dtype == _F32:
        return (np.fmax if opcode == "max" else np.fmin).reduce(values, axis=axis)
    return (np.max if opcode == "max" else np.min)(values, axis=axis)


def tree_sum(values: np.ndarray) -> Any:
    """Sum of a power-of-two-length vector in the interpreter's own pairing order."""
    return _tree_reduce(np.asarray(values), "sum")


def _extremum(lhs, rhs, opcode: str, is_float: bool):
    pick = np.where(lhs > rhs, lhs, rhs) if opcode == "maximum" else np.where(lhs < rhs, lhs, rhs)
    if is_float:
        pick = np.where(np.isnan(lhs), lhs, np.where(np.isnan(rhs), rhs, pick))
    return pick


class Interpreter:
    def __init__(self, ssa_text: str, args: dict[str, Any]) -> None:
        self.program = parse(ssa_text)
        self.memory = {
            name: value.reshape(-1) for name, value in args.items() if isinstance(value, np.ndarray)
        }
        self.scalars = {
            name: (_INT(value) if isinstance(value, (int, np.integer)) else _F32(value))
            for name, value in args.items()
            if not isinstance(value, np.ndarray)
        }

    def run(self, grid: tuple[int, ...]) -> None:
        grid = tuple(grid) + (1,) * (3 - len(grid))
        self.grid = grid
        for pid in itertools.product(*(range(g) for g in grid)):
            self._exec(self.program, {}, pid)

    # -- operands -----------------------------------------------------------------

    def _value(self, token: str, env: dict[int, Any]):
        if token == "none":
            return None
        if token.startswith("%"):
            return env[int(token[1:])]
        if token in self.memory:
            return _Ptr(token, _INT(0))
        if token in self.scalars:
            return self.scalars[token]
        if token in ("inf", "-inf", "nan"):
            return _F32(float(token))
        literal = ast.literal_eval(token)
        if isinstance(literal, bool):
            return np.bool_(literal)
        return _INT(literal) if isinstance(literal, int) else _F32(literal)

    @staticmethod
    def _cast(value, element: str):
        dtype = {"i32": _INT, "f32": _F32, "bf16": _F32, "f16": _F32, "f8e4m3": _F32, "f8e5m2": _F32, "bool": np.bool_}[element]
        return np.asarray(value).astype(dtype) if np.ndim(value) else dtype(value)

    # -- statements ---------------------------------------------------------------

    def _exec(self, ops: list[Any], env: dict[int, Any], pid) -> None:
        for op in ops:
            if isinstance(op, _Loop):
                self._exec_loop(op, env, pid)
            else:
                self._exec_op(op, env, pid)

    def _exec_loop(self, loop: _Loop, env, pid) -> None:
        start, stop, step = (int(self._value(t, env)) for t in loop.bounds)
        carried = [self._value(init, env) for _, init in loop.carried]
        for k in range(start, stop, step):
            env[loop.index] = _INT(k)
            for (arg, _), value in zip(loop.carried, carried):
                env[arg] = value
            try:
                self._exec(loop.body, env, pid)
            except _LeaveLoop:
                break                     # results: the carried values as the iteration found them
            carried = [self._value(t, env) for t in loop.yields]
        for result, value in zip(loop.results, carried):
            env[result] = value

    def _exec_op(self, op: _Op, env, pid) -> None:
        code = op.opcode
        args = [self._value(t, env) for t in op.operands]
        if code == "store":
            self._store(*args)
            return
        if code == "atomic_add":
            self._store(*args, accumulate=True)
            return
        if code == "break_unless":
            if not bool(args[0]):
                raise _LeaveLoop
            return
        shape, element = _parse_type(op.ty)
        (target,) = op.results
        with np.errstate(all="ignore"):
            env[target] = self._compute(code, args, op.attrs, shape, element, pid)

    def _compute(self, code, args, attrs, shape, element, pid):
        if code == "program_id":
            return _INT(pid[attrs["axis"]])
        if code == "num_programs":
            return _INT(self.grid[attrs["axis"]])
        if code == "trans":
            return np.ascontiguousarray(np.transpose(args[0]))
        if code == "arange":
            return np.arange(attrs["start"], attrs["end"], dtype=_INT)
        if code in ("zeros", "empty"):
            return np.zeros(shape, dtype={"i32": _INT, "f32": _F32, "bool": np.bool_}[element])
        if code == "full":
            return np.broadcast_to(self._cast(args[0], element), shape).copy()
        if code == "expand_dims":
            return np.expand_dims(args[0], attrs["axis"])
        if code == "addptr":
            base, offset = args
            index = base.index + offset
            return _Ptr(base.base, np.asarray(index, dtype=_INT) if np.ndim(index) else _INT(index))
        if code == "load":
            return self._load(args[0], args[1], args[2], shape, element)
        if code == "rem":
            lhs64, rhs64 = np.asarray(args[0], dtype=np.int64), np.asarray(args[1], dtype=np.int64)
            return self._cast(np.fmod(lhs64, rhs64).astype(_INT), "i32")     # C remainder
        if code in ("add", "sub", "mul", "div"):
            lhs, rhs = args
            if element == "i32":
                lhs64, rhs64 = np.asarray(lhs, dtype=np.int64), np.asarray(rhs, dtype=np.int64)
                if code == "div":
                    out = np.fix(lhs64 / rhs64).astype(np.int64)
                else:
                    out = {"add": lhs64 + rhs64, "sub": lhs64 - rhs64, "mul": lhs64 * rhs64}[code]
                return self._cast(out.astype(np.int64).astype(_INT), "i32")
            lhs, rhs = self._cast(lhs, "f32"), self._cast(rhs, "f32")
            out = {"add": np.add, "sub": np.subtract, "mul": np.multiply, "div": np.divide}[code](lhs, rhs)
            return self._cast(out, "f32")
        if code == "cmp_lt":
            lhs, rhs = args
            if any(np.asarray(x).dtype == _F32 for x in (lhs, rhs)):
                lhs, rhs = self._cast(lhs, "f32"), self._cast(rhs, "f32")
            return np.less(lhs, rhs)
        if code == "and":
            return np.logical_and(args[0], args[1])
        if code in ("maximum", "minimum"):
            lhs, rhs = self._cast(args[0], element), self._cast(args[1], element)
            return self._cast(_extremum(lhs, rhs, code, element == "f32"), element)
        if code == "neg":
            return self._cast(np.negative(args[0]), element)
        if code == "not":
            return np.logical_not(args[0])
        if code == "exp":
            return self._cast(np.exp(self._cast(args[0], "f32")), "f32")
        if code == "abs" and element == "i32":
            return self._cast(np.abs(args[0]), "i32")
        if code in _FLOAT_UNARY:
            return self._cast(_FLOAT_UNARY[code](self._cast(args[0], "f32")), "f32")
        if code == "select":
            cond, yes, no = args
            return self._cast(np.where(cond, self._cast(yes, element), self._cast(no, element)), element)
        if code in ("sum", "max", "min"):
            if "axis" in attrs:                   # rank-2 operand reduced along one axis
                return self._cast(_axis_reduce(np.asarray(args[0]), code, attrs["axis"]), element)
            return _tree_reduce(np.asarray(args[0]), code)
        if code == "dot":
            lhs, rhs, acc = args
            out = np.asarray(lhs, dtype=np.float64) @ np.asarray(rhs, dtype=np.float64)
            if acc is not None:
                out = out + np.asarray(acc, dtype=np.float64)
            return out.astype(_F32)
        raise NotImplementedError(code)

    # -- memory -------------------------------------------------------------------

    def _load(self, ptr: _Ptr, mask, other, shape, element):
        memory = self.memory[ptr.base]
        parts = [np.asarray(ptr.index)] + [np.asarray(x) for x in (mask, other) if x is not None]
        full = np.broadcast_shapes(*(p.shape for p in parts), shape)
        index = np.broadcast_to(np.asarray(ptr.index, dtype=np.int64), full)
        live = np.ones(full, dtype=bool) if mask is None else np.broadcast_to(mask, full)
        fallback = self._cast(0 if other is None else other, element)
        safe = np.where(live, index, 0)
        if live.any():
            assert safe.min() >= 0 and safe.max() < memory.shape[0], "out-of-bounds load"
        out = np.where(live, memory[safe], np.broadcast_to(fallback, full))
        out = self._cast(out, element)
        return out if full else out.reshape(())[()]

    def _store(self, ptr: _Ptr, value, mask, accumulate: bool = False) -> None:
        memory = self.memory[ptr.base]
        parts = [np.asarray(x) for x in (ptr.index, value, mask) if x is not None]
        full = np.broadcast_shapes(*(p.shape for p in parts))
        index = np.broadcast_to(np.asarray(ptr.index, dtype=np.int64), full).reshape(-1)
        data = np.broadcast_to(np.asarray(value).astype(memory.dtype), full).reshape(-1)
        live = (np.ones(full, dtype=bool) if mask is None else np.broadcast_to(mask, full)).reshape(-1)
        if live.any():
            assert index[live].min() >= 0 and index[live].max() < memory.shape[0], "out-of-bounds store"
        if accumulate:
            np.add.at(memory, index[live], data[live])       # repeated indices all count
        else:
            memory[index[live]] = data[live]


def run(ssa_text: str, args: dict[str, Any], grid: tuple[int, ...]) -> None:
    """Execute the kernel described by ``ssa_text`` over ``grid``.

    ``args`` maps runtime parameter names to NumPy arrays (modified in place, any
    shape, C-contiguous float32) or Python/NumPy scalars."""
    Interpreter(ssa_text, args).run(grid)
