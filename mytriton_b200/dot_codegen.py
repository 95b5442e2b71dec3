"""``tl.dot`` K-loops -> a TMA-fed tcgen05 GEMM kernel for sm_100a.

The reference has no ``tl.dot``; its matmuls are per-thread FMA loops that
re-read A and B from global memory for every k (tests/test_ast_runtime_loop.py:22-53,
README.md:385-396).  This module recognises the tiled form

    acc = tl.zeros((BM, BN), tl.float32)
    for k0 in range(0, K, BK):
        a = tl.load(a_ptr + rows[:, None] * lda + (k0 + kk)[None, :], mask=..., other=0.0)
        b = tl.load(b_ptr + (k0 + kk)[:, None] * ldb + cols[None, :], mask=..., other=0.0)
        acc = tl.dot(a, b, acc)
    tl.store(c_ptr + rows[:, None] * ldc + cols[None, :], acc, mask=...)

by evaluating every index expression *symbolically* (polynomials over program
ids, the loop index, tile coordinates and runtime scalars) and comparing with
the dense-tile form; anything that does not match exactly is left to the SIMT
path.  A match is lowered to one persistent, warp-specialised kernel:

  warp 0      TMA producer: per k-block, one 128B-swizzled box of A (K-major)
              and BN/64 boxes of B (N-major, i.e. the "MN-major" UMMA operand),
              completion counted on an mbarrier per pipeline stage; no multicast.
  warp 1      allocates TMEM, then a single lane issues tcgen05.mma
              (cta_group::1, kind::f16, bf16 x bf16 -> fp32 in TMEM), committing
              each stage back to the producer and each finished tile to the
              epilogue.  Two accumulators (2 x BN columns) let tile i+1's
              mainloop overlap tile i's epilogue.
  warps 2-5   epilogue: tcgen05.ld 32 lanes x 32 columns at a time, the fused
              post-loop elementwise work on those registers, then a 128B-swizzled
              staging box and a TMA store of fp32 C (clipped at the matrix edge by
              the tensor map), optionally to several destinations: this GPU's C and
              the same rows of its peers' C.

The default variant pairs two CTAs on a 256 x BN tile (dot_codegen_pair.py).

Every wait is bounded: when a limit is exceeded the kernel records a code in the
caller's status word, raises a CTA-wide abort flag, lets in-flight copies land,
frees its TMEM and returns.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Any

from .nodes import Const, Param
from .ssa import SSAForRange, SSAItem, SSAOp, SSAOperand, SSAValue
from .types import BF16, BYTE_WIDTH, F16, F32, FLOAT_UNARY, HALF_WIDTH, I32, BlockType, PointerType, shape_of

# --------------------------------------------------------------------------- symbolic polynomials

Monomial = tuple[str, ...]


class Poly:
    """Integer polynomial over named symbols (sorted-tuple monomials -> coefficient)."""

    __slots__ = ("terms",)

    def __init__(self, terms: dict[Monomial, int] | None = None) -> None:
        self.terms = {m: c for m, c in (terms or {}).items() if c != 0}

    @staticmethod
    def const(value: int) -> "Poly":
        return Poly({(): int(value)})

    @staticmethod
    def sym(name: str) -> "Poly":
        return Poly({(name,): 1})

    def __add__(self, other: "Poly") -> "Poly":
        out = dict(self.terms)
        for m, c in other.terms.items():
            out[m] = out.get(m, 0) + c
        return Poly(out)

    def __neg__(self) -> "Poly":
        return Poly({m: -c for m, c in self.terms.items()})

    def __sub__(self, other: "Poly") -> "Poly":
        return self + (-other)

    def __mul__(self, other: "Poly") -> "Poly":
        out: dict[Monomial, int] = {}
        for m1, c1 in self.terms.items():
            for m2, c2 in other.terms.items():
                m = tuple(sorted(m1 + m2))
                out[m] = out.get(m, 0) + c1 * c2
        return Poly(out)

    def __eq__(self, other: object) -> bool:
        return isinstance(other, Poly) and self.terms == other.terms

    def __hash__(self) -> int:
        return hash(frozenset(self.terms.items()))

    def rename(self, mapping: dict[str, str]) -> "Poly":
        return Poly({tuple(sorted(mapping.get(s, s) for s in m)): c for m, c in self.terms.items()})

    def symbols(self) -> set[str]:
        return {s for m in self.terms for s in m}

    def substitute(self, symbol: str, replacement: "Poly") -> "Poly":
        """The polynomial with every occurrence of ``symbol`` replaced by ``replacement``."""
        out = Poly()
        for monomial, coefficient in self.terms.items():
            term = Poly.const(coefficient)
            for factor in monomial:
                term = term * (replacement if factor == symbol else Poly.sym(factor))
            out = out + term
        return out

    def __repr__(self) -> str:
        return " + ".join(f"{c}*{'*'.join(m) or '1'}" for m, c in sorted(self.terms.items())) or "0"


@dataclass(frozen=True)
class Bound:
    """``lhs < rhs`` with both sides polynomials."""

    lhs: Poly
    rhs: Poly


class _Unsupported(Exception):
    pass


class _Symbolic:
    """Evaluates integer/boolean SSA values to polynomials / conjunctions of bounds.

    Coordinate symbols: rank-1 values vary in ``v``; rank-2 values in ``r`` (axis 0)
    and ``c`` (axis 1)."""

    _COORDINATES = {"r", "c", "v", "k"}

    def __init__(self, wraps_enabled: bool = False) -> None:
        self.values: dict[int, Any] = {}
        self.wraps_enabled = wraps_enabled
        self.wrapped_ids: set[int] = set()
        # program-uniform integers that are no polynomial of the program ids (`pid // n`,
        # `pid % n`, `min(a, b)`): each gets a symbol "s:<n>"; what it stands for is kept so
        # that the launcher can evaluate it for every program of a grid
        self.opaque: dict[str, tuple[str, Poly, Poly]] = {}
        self._opaque_names: dict[tuple[str, Poly, Poly], str] = {}
        # index blocks taken modulo a scalar (`offs_m % M`, which keeps the addresses of a ragged
        # tile inside the array without a mask): (the index, the modulus).  The value is carried on
        # as the index itself; the matcher then demands that what wrapped around is never stored.
        self.wraps: list[tuple[Poly, str]] = []

    def _opaque_scalar(self, code: str, lhs: Any, rhs: Any) -> Poly:
        if not isinstance(lhs, Poly) or not isinstance(rhs, Poly):
            raise _Unsupported("arithmetic on non-index values")
        if (lhs.symbols() | rhs.symbols()) & self._COORDINATES:
            raise _Unsupported(f"{code} of a per-element index")
        key = (code, lhs, rhs)
        name = self._opaque_names.get(key)
        if name is None:
            name = self._opaque_names[key] = f"s:{len(self._opaque_names)}"
            self.opaque[name] = key
        return Poly.sym(name)

    def operand(self, operand: SSAOperand, want_rank: int | None = None) -> Any:
        if isinstance(operand, Const):
            if type(operand.value) is not int:
                raise _Unsupported("non-integer constant in index arithmetic")
            return Poly.const(operand.value)
        if isinstance(operand, Param):
            if operand.ty != I32:
                raise _Unsupported("non-i32 scalar in index arithmetic")
            return Poly.sym("p:" + operand.name)
        if isinstance(operand, SSAValue):
            if operand.id not in self.values:
                raise _Unsupported(f"{operand} is not an index expression")
            value = self.values[operand.id]
            if want_rank == 2 and len(shape_of(operand.ty)) == 1 and isinstance(value, Poly):
                return value.rename({"v": "c"})     # NumPy right-aligned broadcast
            return value
        raise _Unsupported("missing operand")

    def visit(self, op: SSAOp) -> None:
        result = op.result
        if result is None:
            return
        rank = len(shape_of(result.ty))
        code = op.opcode
        try:
            if code == "program_id":
                value: Any = Poly.sym(f"pid{op.attrs['axis']}")
            elif code == "arange":
                value = Poly.const(op.attrs["start"]) + Poly.sym("v")
            elif code == "expand_dims":
                inner = self.operand(op.operands[0])
                value = inner.rename({"v": "r" if op.attrs["axis"] == 1 else "c"})
            elif code in ("add", "sub", "mul"):
                lhs, rhs = (self.operand(x, rank) for x in op.operands)
                if not isinstance(lhs, Poly) or not isinstance(rhs, Poly):
                    raise _Unsupported("arithmetic on non-index values")
                value = lhs + rhs if code == "add" else lhs - rhs if code == "sub" else lhs * rhs
            elif code in ("div", "rem", "minimum", "maximum") and rank == 0 and result.ty == I32:
                lhs, rhs = (self.operand(x, rank) for x in op.operands)
                value = self._opaque_scalar(code, lhs, rhs)
            elif code == "trans":
                inner = self.operand(op.operands[0])
                exchange = {"r": "c", "c": "r"}
                if isinstance(inner, Poly):
                    value = inner.rename(exchange)
                elif isinstance(inner, frozenset):
                    value = frozenset(Bound(b.lhs.rename(exchange), b.rhs.rename(exchange)) for b in inner)
                else:
                    raise _Unsupported("transpose of something other than an index block or a mask")
            elif code == "rem" and rank >= 1 and self.wraps_enabled:
                # (only on the matcher's second attempt: otherwise a block remainder is ordinary
                # elementwise work, e.g. `rows % 5` in an epilogue)
                lhs, rhs = (self.operand(x, rank) for x in op.operands)
                modulus = _scalar_symbol(rhs) if isinstance(rhs, Poly) else None
                if not isinstance(lhs, Poly) or modulus is None or not modulus.startswith("p:"):
                    raise _Unsupported("remainder of an index block by something other than a scalar argument")
                self.wraps.append((lhs, modulus))
                self.wrapped_ids.add(result.id)
                value = lhs
            elif code == "cmp_lt":
                lhs, rhs = (self.operand(x, rank) for x in op.operands)
                value = frozenset({Bound(lhs, rhs)})
            elif code == "not" and rank == 0:
                inner = self.operand(op.operands[0])
                if not isinstance(inner, frozenset) or len(inner) != 1:
                    raise _Unsupported("negation of something other than one comparison")
                (bound,) = inner                      # integers: not (a < b) is b < a + 1
                value = frozenset({Bound(bound.rhs, bound.lhs + Poly.const(1))})
            elif code == "and":
                lhs, rhs = (self.operand(x, rank) for x in op.operands)
                if not isinstance(lhs, frozenset) or not isinstance(rhs, frozenset):
                    raise _Unsupported("& of non-comparisons")
                value = lhs | rhs
            elif code == "addptr":
                base, offset = op.operands
                offset_poly = self.operand(offset, rank)
                if isinstance(base, Param):
                    value = (base, offset_poly)
                else:
                    inner_base, inner_offset = self.operand(base, rank)
                    value = (inner_base, inner_offset + offset_poly)
            else:
                return
        except _Unsupported:
            return
        self.values[result.id] = value


# --------------------------------------------------------------------------- the match


@dataclass
class GemmMatch:
    a: Param
    b: Param
    c: Param
    bm: int
    bn: int
    bk: int
    axis_m: int
    axis_n: int
    lda: str          # symbol ("p:<name>") or "#<int>" for the row strides / extents
    ldb: str
    ldc: str
    k_extent: str
    m_extent: str | None
    n_extent: str | None
    epilogue: tuple[str, ...] = ()     # C statements applied per element: acc, row, col -> acc
    operand: str = "bf16"              # element type of A and B: "bf16", "f16", "f8e4m3" or "tf32" (fp32 in memory)
    out: str = "f32"                   # element type of C: "f32" or "bf16" (rounded to nearest even)
    program_tile: tuple[int, int] | None = None    # (BM, BN) of one program, when it differs from the kernel's tile
    c_transposed: bool = False         # C is stored as its transpose: element (row, col) at col * ldc + row
    tile_map: "TileMap | None" = None  # how a program finds its tile, when that is not (pid[axis_m], pid[axis_n])
    b_transposed: bool = False         # B is stored as its transpose [N, K]: element (k, col) at col * ldb + k
    a_transposed: bool = False         # A is stored as its transpose [K, M]: element (row, k) at k * lda + row


@dataclass(frozen=True)
class TileMap:
    """Program -> tile, for launches that do not use one grid axis per tile axis: the tile row and
    column as polynomials over program ids, scalar parameters and opaque scalars (``pid // n``,
    ``pid % n``, ``min``), and the conditions under which a program does any work at all (an early
    ``return``).  The kernel is a dense GEMM over C exactly when the programs that pass the guards
    visit every tile of a rectangle once; that is checked per launch, on the host, by evaluating
    these expressions for every program of the grid."""

    row_tile: Poly
    col_tile: Poly
    guards: tuple[Bound, ...]
    opaque: tuple[tuple[str, tuple[str, Poly, Poly]], ...]


def _scalar_symbol(poly: Poly) -> str | None:
    """A polynomial that is exactly one runtime scalar, or one integer constant."""
    if len(poly.terms) == 1:
        (mono, coef), = poly.terms.items()
        if mono == () :
            return f"#{coef}"
        if len(mono) == 1 and coef == 1 and mono[0].startswith("p:"):
            return mono[0]
    if not poly.terms:
        return "#0"
    return None


def _sym_poly(symbol: str) -> Poly:
    return Poly.const(int(symbol[1:])) if symbol.startswith("#") else Poly.sym(symbol)


def _split_linear(poly: Poly, coord: str) -> tuple[Poly, Poly] | None:
    """poly == stride * coord + rest, with ``coord`` absent from stride and rest."""
    stride, rest = Poly(), Poly()
    for mono, coef in poly.terms.items():
        count = mono.count(coord)
        if count == 0:
            rest = rest + Poly({mono: coef})
        elif count == 1:
            reduced = list(mono)
            reduced.remove(coord)
            stride = stride + Poly({tuple(reduced): coef})
        else:
            return None
    return stride, rest


def _divide(poly: Poly, divisor: Poly) -> Poly | None:
    """poly / divisor when the divisor is an integer constant or a single symbol and the
    division is exact term by term, else None."""
    if len(divisor.terms) != 1:
        return None
    (monomial, coefficient), = divisor.terms.items()
    out: dict[Monomial, int] = {}
    for mono, coef in poly.terms.items():
        if coef % coefficient:
            return None
        remaining = list(mono)
        for factor in monomial:
            if factor not in remaining:
                return None
            remaining.remove(factor)
        out[tuple(remaining)] = coef // coefficient
    return Poly(out)


def _blocks_to_depth(value: Any, bk: int) -> Any:
    """A value of the loop body with the k-block index ``i`` rewritten as ``k / BK``: every term
    that holds ``i`` must hold it once, with a coefficient BK divides (``i * BK * stride``,
    ``K - i * BK``); anything else is no dense K-loop."""
    if isinstance(value, tuple):
        return (value[0], _blocks_to_depth(value[1], bk))
    if isinstance(value, frozenset):
        return frozenset(Bound(_blocks_to_depth(b.lhs, bk), _blocks_to_depth(b.rhs, bk)) for b in value)
    if not isinstance(value, Poly):
        return value
    out: dict = {}
    for monomial, coefficient in value.terms.items():
        uses = monomial.count("i")
        if uses:
            if uses > 1 or coefficient % bk:
                raise _Unsupported("the k-block index is used other than as index * BK")
            coefficient //= bk
            monomial = tuple(sorted("k" if symbol == "i" else symbol for symbol in monomial))
        out[monomial] = out.get(monomial, 0) + coefficient
    return Poly(out)


def _match_tile(offset: Poly, row_coord_extra: Poly | None = None):
    """offset == row * ld + col with row = f(r), col = g(c): returns (row, ld, col)."""
    split_r = _split_linear(offset, "r")
    if split_r is None:
        return None
    ld, rest = split_r
    ld_symbol = _scalar_symbol(ld)
    if ld_symbol is None or "c" in ld.symbols():
        return None
    split_c = _split_linear(rest, "c")
    if split_c is None or split_c[0] != Poly.const(1):
        return None
    base = split_c[1]                       # = row0 * ld + col0, free of r and c
    return ld_symbol, base


def match_gemm_loop(ssa_ops: list[SSAItem], params: list[Param]) -> GemmMatch | None:
    # Second attempt: index blocks taken modulo a scalar argument (`offs_m % M`) read as the index
    # itself, under the conditions _match then checks.  Only when the plain reading fails, so that a
    # remainder which is ordinary elementwise work stays one.
    for wraps_enabled in (False, True):
        try:
            match = _match(ssa_ops, wraps_enabled)
        except _Unsupported:
            match = None
        if match is not None:
            return match
    return None


def _uses_wrapped_index(ssa_ops: list[SSAItem], wrapped: set[int], roots: list[SSAOperand]) -> bool:
    """Whether any of ``roots`` is computed from an index block that was read through a remainder —
    other than through a load, whose data is what the wrap is allowed to affect."""
    tainted = set(wrapped)
    producers: dict[int, SSAOp] = {}

    def scan(items) -> None:
        for item in items:
            if isinstance(item, SSAForRange):
                scan(item.body)
            elif item.result is not None:
                producers[item.result.id] = item
                if item.opcode != "load" and any(
                        isinstance(x, SSAValue) and x.id in tainted for x in item.operands):
                    tainted.add(item.result.id)

    scan(ssa_ops)
    return any(isinstance(root, SSAValue) and root.id in tainted for root in roots)


def _match(ssa_ops: list[SSAItem], wraps_enabled: bool = False) -> GemmMatch | None:
    loops = [op for op in ssa_ops if isinstance(op, SSAForRange)]
    stores = [op for op in ssa_ops if isinstance(op, SSAOp) and op.opcode == "store"]
    if len(loops) != 1 or len(stores) != 1:
        return None
    loop, store = loops[0], stores[0]
    if ssa_ops.index(store) < ssa_ops.index(loop):
        return None
    if not loop.results or any(isinstance(op, SSAForRange) for op in loop.body):
        return None
    if any(op.opcode == "store" for op in loop.body):
        return None

    sym = _Symbolic(wraps_enabled)
    zeros_ids = set()
    value_ops: list[SSAOp] = []               # non-index work outside the loop: the epilogue
    for op in ssa_ops:
        if isinstance(op, SSAForRange) or op.opcode == "store":
            continue
        if op.opcode in ("sum", "max", "min", "dot") or op.result is None:
            return None                       # a reduction, or a side effect other than the one store
        if op.opcode == "zeros":
            zeros_ids.add(op.result.id)
            continue
        sym.visit(op)
        if op.result.id not in sym.values or op.opcode == "load":
            value_ops.append(op)

    # loop header: range(0, K, BK), or range(0, cdiv(K, BK)) whose index counts k-blocks; one
    # carried fp32 accumulator initialised to zeros
    if not (isinstance(loop.start, Const) and loop.start.value == 0 and isinstance(loop.step, Const)):
        return None
    bk = loop.step.value
    counts_blocks = False
    stop = sym.operand(loop.stop)
    k_extent = _scalar_symbol(stop) if isinstance(stop, Poly) else None
    if bk == 1 and isinstance(stop, Poly) and len(stop.terms) == 1 and stop.symbols() <= set(sym.opaque):
        # (K + BK - 1) // BK trips: the index is k / BK, and must only occur as index * BK
        ((monomial, coefficient),) = stop.terms.items()
        code, dividend, divisor = sym.opaque[monomial[0]] if len(monomial) == 1 else (None, None, None)
        if code == "div" and coefficient == 1 and not divisor.symbols() and divisor.terms.get((), 0) > 1:
            bk = divisor.terms[()]
            k_extent = _scalar_symbol(dividend - Poly.const(bk - 1))
            counts_blocks = True
    if k_extent is None:
        return None
    slots = list(zip(loop.carried_inputs, loop.carried_args, loop.yields, loop.results))
    accumulators = [slot for slot in slots
                    if isinstance(slot[0], SSAValue) and slot[0].id in zeros_ids]
    if len(accumulators) != 1:
        return None
    initial, arg, yielded, result = accumulators[0]
    acc_ty = result.ty
    if not isinstance(acc_ty, BlockType) or acc_ty.rank != 2 or acc_ty.element != F32:
        return None
    bm, bn = acc_ty.shape

    sym.values[loop.index.id] = Poly.sym("i" if counts_blocks else "k")
    # Every other carried value must be an induction value: a pointer or index block that each
    # iteration advances by a loop-invariant amount (`a_ptrs += BK`, `b_ptrs += BK * N`).  With the
    # loop counting k = 0, BK, 2 BK, ... its value at the top of an iteration is start + k * (step / BK).
    producers = {op.result.id: op for op in loop.body if op.result is not None}
    for op in loop.body:
        sym.visit(op)                         # first pass: the loop-invariant amounts (`BK * N`)
    for slot in slots:
        if slot is accumulators[0]:
            continue
        slot_initial, slot_arg, slot_yield, slot_result = slot
        step_op = producers.get(slot_yield.id) if isinstance(slot_yield, SSAValue) else None
        if step_op is None or step_op.opcode not in ("addptr", "add") or step_op.operands[0] != slot_arg:
            return None
        try:
            advance = sym.operand(step_op.operands[1])
            start_value = sym.operand(slot_initial)
        except _Unsupported:
            return None
        if not isinstance(advance, Poly) or advance.symbols() & {"r", "c", "v", "k"}:
            return None
        if any(coefficient % bk for coefficient in advance.terms.values()):
            return None
        per_k = Poly({monomial: coefficient // bk for monomial, coefficient in advance.terms.items()})
        if step_op.opcode == "addptr" and isinstance(start_value, tuple):
            sym.values[slot_arg.id] = (start_value[0], start_value[1] + Poly.sym("k") * per_k)
        elif step_op.opcode == "add" and isinstance(start_value, Poly):
            sym.values[slot_arg.id] = start_value + Poly.sym("k") * per_k
        else:
            return None
        if any(isinstance(op, SSAOp) and any(x == slot_result for x in op.operands)
               for op in ssa_ops if not isinstance(op, SSAForRange)):
            return None                       # the advanced value is read after the loop
    loads: dict[int, SSAOp] = {}
    dots: list[SSAOp] = []
    transposes: dict[int, SSAOperand] = {}    # tl.trans(loaded tile): result id -> the tile
    for op in loop.body:
        if op.opcode == "load":
            loads[op.result.id] = op
        elif op.opcode == "dot":
            dots.append(op)
        elif op.opcode == "trans" and op.result is not None and not isinstance(sym.values.get(
                getattr(op.operands[0], "id", None)), (Poly, frozenset)):
            transposes[op.result.id] = op.operands[0]
            continue
        elif op.opcode in ("sum", "max", "min", "exp", "div", "select", "maximum", "minimum", "neg") \
                or op.opcode in FLOAT_UNARY:
            return None
        sym.visit(op)
    if len(dots) != 1 or len(loads) != 2:
        return None
    if counts_blocks:
        # from the block count i to the depth k = i * BK the rest of the matcher works in
        body_ids = {op.result.id for op in loop.body if op.result is not None}
        for value_id in body_ids & set(sym.values):
            sym.values[value_id] = _blocks_to_depth(sym.values[value_id], bk)
    dot = dots[0]
    a_val, b_val, acc_in = dot.operands
    if acc_in is None:
        # `acc += tl.dot(a, b)`: the product feeds exactly one add with the carried accumulator
        users = [op for op in loop.body if any(x == dot.result for x in op.operands)]
        if len(users) != 1 or users[0].opcode != "add" or users[0].result != yielded:
            return None
        if sorted(map(repr, users[0].operands)) != sorted(map(repr, (arg, dot.result))):
            return None
        if sum(any(x == arg for x in op.operands) for op in loop.body) != 1:
            return None
    elif acc_in != arg or yielded != dot.result:
        return None
    elif sum(any(x == arg for x in op.operands) for op in loop.body) != 1:
        return None                           # the accumulator is read by something besides the dot
    if not (isinstance(a_val, SSAValue) and isinstance(b_val, SSAValue)):
        return None
    # an operand may be the transpose of a loaded tile (`tl.dot(q, tl.trans(k))`): the tile is then
    # read with its two coordinates exchanged
    a_source, b_source = transposes.get(a_val.id, a_val), transposes.get(b_val.id, b_val)
    a_flipped, b_flipped = a_source is not a_val, b_source is not b_val
    if not (isinstance(a_source, SSAValue) and isinstance(b_source, SSAValue)):
        return None
    if a_source.id not in loads or b_source.id not in loads or a_source.id == b_source.id:
        return None
    a_load, b_load = loads[a_source.id], loads[b_source.id]
    operand_type = a_val.ty.element if isinstance(a_val.ty, BlockType) else None
    tf32 = operand_type == F32 and dot.attrs.get("input_precision") == "tf32"
    if operand_type not in HALF_WIDTH + BYTE_WIDTH and not tf32:
        return None                           # fp32 operands: SIMT path (no silent tf32 rounding)
    if a_val.ty != BlockType((bm, bk), operand_type) or b_val.ty != BlockType((bk, bn), operand_type):
        return None

    exchange = {"r": "c", "c": "r"}

    def tile_of(load: SSAOp, flipped: bool, stored_transposed: bool):
        """The operand's tile in the coordinates of the dot's operand.  ``flipped``: the operand is
        tl.trans of what was loaded, so the load's coordinates are exchanged first (its mask too);
        ``stored_transposed``: try the tile as c * ld + r instead of r * ld + c."""
        ptr, mask, other = load.operands
        if other is not None and not (isinstance(other, Const) and other.value == 0):
            return None
        if not isinstance(ptr, SSAValue) or ptr.id not in sym.values:
            return None
        base, offset = sym.values[ptr.id]
        if flipped:
            offset = offset.rename(exchange)
        tile = _match_tile(offset.rename(exchange) if stored_transposed else offset)
        if tile is None:
            return None
        bounds = None
        if mask is not None:
            if not isinstance(mask, SSAValue) or not isinstance(sym.values.get(mask.id), frozenset):
                return None
            bounds = sym.values[mask.id]
            if flipped:
                bounds = frozenset(Bound(b.lhs.rename(exchange), b.rhs.rename(exchange)) for b in bounds)
        return base, tile[0], tile[1], bounds

    a_tile, b_tile = tile_of(a_load, a_flipped, False), tile_of(b_load, b_flipped, False)
    a_transposed = b_transposed = False
    if a_tile is None:
        # A stored as its transpose, [K, M] row-major (x.T @ y, the weight gradient of a linear
        # layer): element (r, c) of the [BM, BK] operand at c * lda + r
        a_tile = tile_of(a_load, a_flipped, True)
        a_transposed = True
    if a_tile is not None and b_tile is None:
        # B stored as its transpose, [N, K] row-major (a weight matrix applied as x @ W.T): element
        # (r, c) of the [BK, BN] operand at c * ldb + r
        b_tile = tile_of(b_load, b_flipped, True)
        b_transposed = True
    if a_tile is None or b_tile is None:
        return None
    a_param, lda, a_base, a_bounds = a_tile
    b_param, ldb, b_base, b_bounds = b_tile

    # store: the loop result, written as a dense [BM,BN] tile
    c_ptr, c_value, c_mask = store.operands
    if not isinstance(c_value, SSAValue) or not isinstance(c_ptr, SSAValue) or c_ptr.id not in sym.values:
        return None
    c_param, c_offset = sym.values[c_ptr.id]
    c_tile = _match_tile(c_offset)
    c_transposed = False
    if c_tile is None:
        # C stored as its transpose: element (r, c) of the tile at c * ldc + r
        c_tile = _match_tile(c_offset.rename({"r": "c", "c": "r"}))
        c_transposed = True
    if c_tile is None:
        return None
    ldc, c_base = c_tile
    c_bounds = None
    if c_mask is not None:
        if not isinstance(c_mask, SSAValue) or not isinstance(sym.values.get(c_mask.id), frozenset):
            return None
        c_bounds = sym.values[c_mask.id]
    if (c_param.ty not in (PointerType(F32), PointerType(BF16), PointerType(F16))
            or a_param.ty != PointerType(operand_type)
            or b_param.ty != PointerType(operand_type)):
        return None

    # where a program's tile starts: a_base = row0 * lda + k, b_base = k * ldb + col0, and C
    # at row0 * ldc + col0 (col0 * ldc + row0 when it is stored transposed)
    k = Poly.sym("k")
    row0 = a_base - k * _sym_poly(lda) if a_transposed else _divide(a_base - k, _sym_poly(lda))
    col0 = _divide(b_base - k, _sym_poly(ldb)) if b_transposed else b_base - k * _sym_poly(ldb)
    if col0 is None:
        return None
    if row0 is None or (row0.symbols() | col0.symbols()) & _Symbolic._COORDINATES:
        return None
    if c_base != (col0 * _sym_poly(ldc) + row0 if c_transposed else row0 * _sym_poly(ldc) + col0):
        return None
    row_tile, col_tile = _divide(row0, Poly.const(bm)), _divide(col0, Poly.const(bn))
    if row_tile is None or col_tile is None:
        return None
    r, c = Poly.sym("r"), Poly.sym("c")
    guards: list[Bound] = []

    def extents(bounds, row_expr: Poly, col_expr: Poly):
        """Masks must be exactly {row < R, col < C} (either may be absent), apart from
        conditions on the program as a whole (an early return), which are collected."""
        row_ext = col_ext = None
        own: set[Bound] = set()
        for bound in bounds or ():
            if not (bound.lhs.symbols() | bound.rhs.symbols()) & _Symbolic._COORDINATES:
                own.add(Bound(bound.lhs - bound.rhs, Poly()))      # a guard, as `difference < 0`
                continue
            # `coordinate < extent` in any arrangement of its terms (`cols < K - k0` bounds k0 + cols by K)
            difference = bound.lhs - bound.rhs
            row_symbol = _scalar_symbol(row_expr - difference)
            col_symbol = _scalar_symbol(col_expr - difference)
            if row_symbol is not None:
                row_ext = row_symbol
            elif col_symbol is not None:
                col_ext = col_symbol
            else:
                raise _Unsupported("mask does not bound the tile's own rows/columns")
        return row_ext, col_ext, own

    a_rows, a_cols, a_guards = extents(a_bounds, row0 + r, k + c)
    b_rows, b_cols, b_guards = extents(b_bounds, k + r, col0 + c)
    c_rows, c_cols, c_guards = extents(c_bounds, row0 + r, col0 + c)
    # `offs_m % M` / `offs_n % N` on the operands' indices: rows (columns) past the extent read
    # rows (columns) from the start of the array instead of being masked.  Inside the extent
    # nothing changes, so the kernel is the dense GEMM exactly if the store is masked by that
    # same extent; then the wrap stands for the row (column) mask the loads do not have.
    for wrapped, modulus in sym.wraps:
        by_axis = {wrapped.rename({"v": "r"}): "rows", wrapped.rename({"v": "c"}): "cols"}
        if by_axis.get(row0 + r) == "rows" and c_rows == modulus and a_rows in (None, modulus):
            a_rows = modulus
        elif by_axis.get(col0 + c) == "cols" and c_cols == modulus and b_cols in (None, modulus):
            b_cols = modulus
        else:
            return None
    if not (a_guards <= c_guards and b_guards <= c_guards):
        return None             # a program that loads nothing but still stores is no GEMM tile
    guards = sorted(c_guards, key=repr)
    # one grid axis per tile axis and no guard: the plain case, nothing to check per launch
    axis_m = next((axis for axis in range(3) if row_tile == Poly.sym(f"pid{axis}")), None)
    axis_n = next((axis for axis in range(3) if col_tile == Poly.sym(f"pid{axis}")), None)
    tile_map = None
    if guards or axis_m is None or axis_n is None or axis_m == axis_n:
        allowed = ("pid0", "pid1", "pid2")
        free = {symbol for poly in (row_tile, col_tile, *(g.lhs for g in guards)) for symbol in poly.symbols()}
        if any(not (symbol in allowed or symbol.startswith(("p:", "s:"))) for symbol in free):
            return None
        tile_map = TileMap(row_tile, col_tile, tuple(guards), tuple(sorted(sym.opaque.items())))
        axis_m, axis_n = 0, 1
    if c_transposed and c_param.ty != PointerType(F32):
        return None             # the transposed store is implemented for fp32 C
    for ext in (a_cols, b_rows):
        if ext is not None and ext != k_extent:
            return None
    m_extent = a_rows or c_rows
    n_extent = b_cols or c_cols
    if (a_rows and c_rows and a_rows != c_rows) or (b_cols and c_cols and b_cols != c_cols):
        return None

    atom = 32 if tf32 else 128 if operand_type in BYTE_WIDTH else 64    # elements in one 128-byte swizzle row
    # The programs' tiles only say which part of C the launch covers.  The kernel is proven to
    # be a dense GEMM over that part, so it may be computed in any tiling: a tile this
    # generator implements is kept (BM 128, or 256 = one CTA-pair tile); other tiles of useful
    # size are recomputed in the default 128 x 256 tiling; small ones stay on the SIMT path,
    # which has no alignment demands.
    program_tile = (bm, bn)
    implemented = (bm in (128, 256) and bn % max(64, atom) == 0 and 64 <= bn <= 256
                   and bk % atom == 0 and atom <= bk <= 4 * atom
                   and (bm == 128 or bn % max(128, 2 * atom) == 0))
    if not implemented:
        if bm < 64 or bn < 64 or bk * 2 < atom:
            return None
        bm, bn, bk = 128, 256, atom
    if sym.wrapped_ids:
        # the wrapped indices may address the operands and nothing else: an epilogue, a store
        # address or a store mask computed from them would see `offs % M` as `offs`
        roots = [operand for op in value_ops for operand in op.operands] + [c_ptr, c_mask]
        if _uses_wrapped_index(ssa_ops, sym.wrapped_ids, roots):
            return None
    epilogue = _match_epilogue(value_ops, sym, result, c_value, row0, col0, (m_extent, n_extent))
    return GemmMatch(a_param, b_param, c_param, bm, bn, bk, axis_m, axis_n,
                     lda, ldb, ldc, k_extent, m_extent, n_extent, epilogue,
                     "tf32" if tf32 else operand_type.name, c_param.ty.element.name, program_tile,
                     c_transposed, tile_map, b_transposed, a_transposed)


_EPILOGUE_OPS = {"add", "sub", "mul", "div", "rem", "maximum", "minimum", "neg", "not", "exp", "select", "cmp_lt",
                 "and", *FLOAT_UNARY}


def _match_epilogue(value_ops: list[SSAOp], sym: _Symbolic, loop_result: SSAValue,
                    stored: SSAValue, row0: Poly, col0: Poly,
                    extents: tuple[str | None, str | None] = (None, None)) -> tuple[str, ...]:
    """Elementwise work between the K-loop and the store, as C statements over
    ``acc`` (the accumulator element), ``row`` and ``col``.

    Operands may be the accumulator, earlier epilogue values, constants, scalar
    parameters, row/column vectors loaded from ``ptr + rows`` / ``ptr + cols`` (a bias,
    a per-row scale), and integer index expressions in the element's global row and
    column (``offs_m[:, None] < offs_n[None, :]`` for a triangular mask).  Raises
    _Unsupported for anything else, which sends the whole kernel to the SIMT path."""
    from .cuda_codegen import SSACUDACodegen

    text = SSACUDACodegen()
    names: dict[int, str] = {loop_result.id: "acc"}
    pending: dict[int, tuple[str, Param]] = {}        # rank-1 loads awaiting their expand_dims
    lines: list[str] = []
    r, c, v = Poly.sym("r"), Poly.sym("c"), Poly.sym("v")

    def vector_kind(offset: Poly, rank: int) -> str:
        coordinate = {1: (v, v), 2: (r, c)}[rank]
        if offset == row0 + coordinate[0]:
            return "row"
        if offset == col0 + coordinate[1]:
            return "col"
        raise _Unsupported("epilogue load is not a row or column vector of the tile")

    def read(kind: str, param: Param) -> str:
        index, extent = ("row", "m_rows") if kind == "row" else ("col", "n_cols")
        element = f"{param.name}[{index}]"
        if param.ty.element == BF16:
            element = f"__uint_as_float(((unsigned)({element})) << 16)"
        elif param.ty.element == F16:
            element = f"mtb_half_bits_to_float({element})"
        return f"({index} < {extent} ? {element} : 0.0f)"

    def index_text(poly: Poly, operand_rank: int, consumer_rank: int) -> str:
        """An index polynomial as a C int expression in ``row`` and ``col``: the tile-local
        coordinates are replaced by global ones, after which no program id may remain."""
        if operand_rank == 1:
            if consumer_rank != 2:
                raise _Unsupported("rank-1 index value outside a tile expression")
            poly = poly.rename({"v": "c"})              # NumPy right-aligned broadcast
        poly = poly.substitute("r", Poly.sym("row") - row0).substitute("c", Poly.sym("col") - col0)
        parts = []
        for monomial, coefficient in sorted(poly.terms.items()):
            factors = [str(coefficient)] if coefficient != 1 or not monomial else []
            for symbol in monomial:
                if symbol in ("row", "col"):
                    factors.append(symbol)
                elif symbol.startswith("p:"):
                    factors.append(symbol[2:])
                elif symbol in sym.opaque:
                    factors.append(uniform_text(symbol))
                else:
                    raise _Unsupported(f"index expression keeps {symbol} per element")
            parts.append(" * ".join(factors))
        return "(" + " + ".join(parts or ["0"]) + ")"

    def uniform_text(symbol: str) -> str:
        """A program-uniform integer that is no polynomial (``M % 3``, ``min(M, N)``) as C.  Its
        operands hold no tile coordinate, so rendering them substitutes nothing; one that depends
        on a program id has no meaning per element and is refused by ``index_text``."""
        code, lhs, rhs = sym.opaque[symbol]
        a, b = index_text(lhs, 0, 0), index_text(rhs, 0, 0)
        return {"div": f"({a} / {b})", "rem": f"({a} % {b})",
                "minimum": f"min({a}, {b})", "maximum": f"max({a}, {b})"}[code]

    def render(operand: SSAOperand, consumer_rank: int) -> str:
        if isinstance(operand, Const):
            return text.literal(operand.value)
        if isinstance(operand, Param):
            if isinstance(operand.ty, PointerType):
                raise _Unsupported("pointer in epilogue arithmetic")
            return operand.name
        if isinstance(operand, SSAValue) and operand.id in names:
            return names[operand.id]
        known = sym.values.get(operand.id) if isinstance(operand, SSAValue) else None
        operand_rank = len(shape_of(operand.ty)) if isinstance(operand, SSAValue) else 0
        if isinstance(known, Poly):
            return index_text(known, operand_rank, consumer_rank)
        if isinstance(known, frozenset):                # a conjunction of index comparisons
            return "(" + " && ".join(
                f"({index_text(bound.lhs, operand_rank, consumer_rank)} < "
                f"{index_text(bound.rhs, operand_rank, consumer_rank)})" for bound in sorted(known, key=repr)
            ) + ")"
        raise _Unsupported(f"epilogue operand {operand} is not available per element")

    for op in value_ops:
        result = op.result
        rank = len(shape_of(result.ty))
        if op.opcode == "load":
            ptr, mask, other = op.operands
            if other is not None and not (isinstance(other, Const) and other.value == 0):
                raise _Unsupported("epilogue load with a non-zero fallback")
            if not isinstance(ptr, SSAValue) or not isinstance(sym.values.get(ptr.id), tuple):
                raise _Unsupported("epilogue load through an unknown pointer")
            param, offset = sym.values[ptr.id]
            if rank not in (1, 2):
                raise _Unsupported("scalar load in a dot epilogue")
            whole = _match_tile(offset) if rank == 2 else None
            if whole is not None and whole[1] == row0 * _sym_poly(whole[0]) + col0:
                # a whole tile of another matrix at the element's own row and column (a residual, the
                # old C of `c += a @ b`): read per element; its mask may only bound rows and columns
                # by the extents the store is bounded by, which is what the read is guarded with
                if mask is not None:
                    bounds = sym.values.get(mask.id) if isinstance(mask, SSAValue) else None
                    if not isinstance(bounds, frozenset):
                        raise _Unsupported("epilogue load mask")
                    for bound in bounds:
                        limit = _scalar_symbol(bound.rhs)
                        wanted = extents[0] if bound.lhs == row0 + r else extents[1] if bound.lhs == col0 + c else None
                        if limit is None or limit != wanted:
                            raise _Unsupported("epilogue tile mask is not the store's own row / column mask")
                ld = whole[0]
                stride = ld[2:] if ld.startswith("p:") else ld[1:]
                element = f"{param.name}[(long long)row * ({stride}) + col]"
                if param.ty.element == BF16:
                    element = f"__uint_as_float(((unsigned)({element})) << 16)"
                elif param.ty.element == F16:
                    element = f"mtb_half_bits_to_float({element})"
                elif param.ty.element != F32:
                    raise _Unsupported("epilogue tiles are read from fp32, bf16 or fp16 arrays")
                names[result.id] = f"((row < m_rows && col < n_cols) ? {element} : 0.0f)"
                continue
            kind = vector_kind(offset, rank)
            if mask is not None:
                bounds = sym.values.get(mask.id) if isinstance(mask, SSAValue) else None
                if not isinstance(bounds, frozenset) or len(bounds) != 1:
                    raise _Unsupported("epilogue load mask")
                (bound,) = bounds
                if bound.lhs != offset or _scalar_symbol(bound.rhs) is None:
                    raise _Unsupported("epilogue load mask does not bound the vector's own index")
            if rank == 1:
                pending[result.id] = (kind, param)
                if kind == "col":                       # a rank-1 vector broadcasts along columns
                    names[result.id] = read(kind, param)
            else:
                names[result.id] = read(kind, param)
        elif isinstance(sym.values.get(result.id), Poly):
            if rank != 1:       # pure index arithmetic; rank-1 values are rendered where a tile uses them
                names[result.id] = index_text(sym.values[result.id], rank, rank)
        elif op.opcode == "expand_dims":
            source = op.operands[0]
            if isinstance(source, SSAValue) and isinstance(sym.values.get(source.id), Poly):
                continue                                # an index vector: used through its polynomial
            if not isinstance(source, SSAValue) or source.id not in pending:
                raise _Unsupported("expand_dims of a non-vector in a dot epilogue")
            kind, param = pending[source.id]
            if (kind, op.attrs["axis"]) not in (("row", 1), ("col", 0)):
                raise _Unsupported("vector expanded along the wrong axis")
            names[result.id] = read(kind, param)
        elif op.opcode in _EPILOGUE_OPS:
            args = [render(operand, rank) for operand in op.operands]
            ctype = {"bool": "bool", "i32": "int", "f32": "float"}.get(element_name(result.ty))
            if ctype is None:
                raise _Unsupported(f"{element_name(result.ty)} values in a dot epilogue")
            name = f"e{result.id}"
            lines.append(f"const {ctype} {name} = {text._expr(op, args, result.ty)};")
            names[result.id] = name
        else:
            raise _Unsupported(f"{op.opcode} in a dot epilogue")
    if stored.id not in names:
        raise _Unsupported("stored value is not derived from the accumulator")
    if stored.id != loop_result.id:
        lines.append(f"acc = {names[stored.id]};")
    return tuple(lines)


def element_name(ty) -> str:
    element = ty.element if isinstance(ty, BlockType) else ty
    return getattr(element, "name", "ptr")


# --------------------------------------------------------------------------- the kernel text

WAIT_LIMIT_CYCLES = 4_000_000_000      # ~2 s at B200 clocks; far above any legitimate wait

_PRELUDE = r'''
struct alignas(64) MtbTensorMap { unsigned long long v[16]; };
struct alignas(64) MtbTensorMaps8 { MtbTensorMap m[8]; };   // C on this GPU and on its peers
#define MTB_DEV static __device__ __forceinline__ __attribute__((unused))
#ifndef MTB_MMA_KIND
#define MTB_MMA_KIND "f16"        // tcgen05.mma .kind: "f16" (fp16/bf16 operands) or "tf32"
#endif

// x.to(tl.float16) / x.to(tl.bfloat16) in a fused epilogue: the value rounded to that precision
static __device__ __forceinline__ __attribute__((unused)) float mtb_round_f16(float f) {
    unsigned short h;
    asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f));
    asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h));
    return f;
}
static __device__ __forceinline__ __attribute__((unused)) float mtb_round_bf16(float f) {
    unsigned short h;
    asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(f));
    return __uint_as_float(((unsigned)h) << 16);
}
// an fp16 element of an epilogue vector or tile, widened
static __device__ __forceinline__ __attribute__((unused)) float mtb_half_bits_to_float(unsigned short h) {
    float f;
    asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h));
    return f;
}

MTB_DEV unsigned mtb_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
MTB_DEV void mtb_mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
MTB_DEV void mtb_mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
MTB_DEV void mtb_mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
MTB_DEV bool mtb_mbar_try(unsigned bar, unsigned parity) {
    unsigned done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
// Bounded wait: gives up after MTB_WAIT_LIMIT cycles (or as soon as another thread
// of the CTA gave up), recording `code` in the caller's status word.
MTB_DEV bool mtb_mbar_wait(unsigned bar, unsigned parity, volatile unsigned* abort_flag,
                           unsigned* status, unsigned code) {
    if (mtb_mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mtb_mbar_try(bar, parity)) {
        if (*abort_flag) return false;
        if (clock64() - t0 > MTB_WAIT_LIMIT) {
            *abort_flag = 1u;
            atomicCAS(status, 0u, code);
            return false;
        }
    }
    return true;
}
MTB_DEV void mtb_tma_load_2d(unsigned dst, const MtbTensorMap* map, unsigned bar, int c_inner, int c_outer) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(dst), "l"((unsigned long long)map), "r"(bar), "r"(c_inner), "r"(c_outer) : "memory");
}
MTB_DEV void mtb_tma_store_2d(const MtbTensorMap* map, unsigned src, int c_inner, int c_outer) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 :: "l"((unsigned long long)map), "r"(src), "r"(c_inner), "r"(c_outer) : "memory");
}
// Shared-memory matrix descriptor, 128-byte swizzle, Blackwell descriptor version.
MTB_DEV unsigned long long mtb_desc(unsigned smem_addr, unsigned lbo_bytes, unsigned sbo_bytes,
                                    unsigned long long layout_type = 2ull) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= layout_type << 61;          // 2: 128-byte swizzle of 16-byte chunks; 1: of 32-byte chunks
    return d;
}
MTB_DEV void mtb_umma_bf16(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                           unsigned idesc, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::" MTB_MMA_KIND " [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
MTB_DEV void mtb_umma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 :: "r"(bar) : "memory");
}
MTB_DEV void mtb_tmem_ld32(unsigned taddr, unsigned (&v)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
                   "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
                   "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
                   "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                   "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
'''

_KERNEL = r'''
extern "C" __global__ __launch_bounds__(192, 1)
void @NAME@(@SIGNATURE@, const __grid_constant__ MtbTensorMap map_a,
            const __grid_constant__ MtbTensorMap map_b,
            const __grid_constant__ MtbTensorMaps8 maps_c, int n_dst,
            int grid_m, int grid_n, int m_rows, int n_cols, int k_depth, int ldc,
            @SPLIT_PARAMS@unsigned* status) {
    constexpr int BM = @BM@, BN = @BN@, BK = @BK@, STAGES = @STAGES@;
    constexpr int EB = @EB@;                          // bytes per operand element (2; 4 for tf32; 1 for fp8)
    constexpr int AE = 128 / EB;                      // elements in one 128-byte swizzle row
    constexpr int UK = 32 / EB;                       // k-depth of one MMA instruction (32 bytes)
    // Split K: the k-blocks of every tile are dealt out to `splits` units of work, kb_per to
    // each; unit t computes k-blocks [split * kb_per, ...) of tile t % (grid_m * grid_n) and
    // stores its raw partial sums `split_rows` rows further down in a workspace, which a second
    // kernel adds up in a fixed order.  Without it there is one unit per tile.
    @SPLIT_DECLS@
    // Rows of A that are fetched.  The MMA always reads 128: when the launch covers fewer rows
    // (a skinny problem) the rest of the operand is whatever shared memory holds there, which
    // only reaches accumulator rows that are never stored, and the freed space buys stages.
    constexpr int A_ROWS = @A_ROWS@;
    constexpr int A_BYTES = A_ROWS * BK * EB;         // BK/AE swizzle atoms of [A_ROWS][AE]
    constexpr int B_BYTES = BK * BN * EB;             // BN/AE sub-tiles of [BK][AE]
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int OUT_BYTES = 32 * 32 * 4;            // one 32-row x 32-column fp32 staging box
    constexpr int TMEM_COLS = @TMEM_COLS@;            // two accumulators of BN columns
    constexpr unsigned AB_FORMAT = @AB_FORMAT@u;     // kind::f16: 0 = fp16, 1 = bf16; kind::tf32: 2; kind::f8f6f4: 0 = e4m3, 1 = e5m2
    // B in memory: [K, N] row-major (the MN-major operand: sub-tiles of [BK][AE]) or its transpose
    // [N, K] (K-major like A: sub-tiles of [BN][AE])
    constexpr bool B_KMAJOR = @B_KMAJOR@;
    // A in memory: [M, K] row-major (K-major: sub-tiles of [A_ROWS][AE]) or its transpose [K, M]
    // (the MN-major operand: sub-tiles of [BK][AE], one per AE rows of the tile)
    constexpr bool A_MMAJOR = @A_MMAJOR@;
    constexpr unsigned IDESC = (1u << 4) | (AB_FORMAT << 7) | (AB_FORMAT << 10)
                             | ((A_MMAJOR ? 1u : 0u) << 15) | ((B_KMAJOR ? 0u : 1u) << 16)
                             | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);

    extern __shared__ unsigned char mtb_dyn_smem[];
    __shared__ unsigned long long bar_full[STAGES], bar_empty[STAGES], bar_acc_full[2], bar_acc_empty[2];
    __shared__ unsigned tmem_slot;
    __shared__ unsigned abort_word;
    volatile unsigned* abort_flag = &abort_word;

    const unsigned tiles_base = (mtb_smem(mtb_dyn_smem) + 1023u) & ~1023u;
    const unsigned out_base = tiles_base + STAGES * STAGE_BYTES;   // 4 warps x 2 boxes
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int base_tiles = grid_m * grid_n;
    const int num_tiles = base_tiles * splits;
    const int num_kb = (k_depth + BK - 1) / BK;

    if (threadIdx.x == 0) {
        abort_word = 0u;
        for (int s = 0; s < STAGES; ++s) { mtb_mbar_init(mtb_smem(&bar_full[s]), 1); mtb_mbar_init(mtb_smem(&bar_empty[s]), 1); }
        for (int s = 0; s < 2; ++s) { mtb_mbar_init(mtb_smem(&bar_acc_full[s]), 1); mtb_mbar_init(mtb_smem(&bar_acc_empty[s]), 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(mtb_smem(&tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = tmem_slot;

    // logical program -> tile coordinates, GROUP_M row-tiles at a time for L2 reuse
    // (a / b for 0 <= a < 2^22, 0 < b: one float division and a correction instead of the ~170
    // cycles of an integer division, which one thread pays several times before its first copy)
    auto quotient = [](int a, int b) {
        if (a >= (1 << 22)) return a / b;             // beyond the range where the estimate is within one
        int q = (int)__fdividef((float)a, (float)b);
        const int r = a - q * b;
        return r < 0 ? q - 1 : (r >= b ? q + 1 : q);
    };
    auto k_range = [&](int t, int& split, int& kb0, int& kb1) {
        split = splits == 1 ? 0 : quotient(t, base_tiles);
        kb0 = split * kb_per;
        kb1 = (num_kb - kb0 < kb_per) ? num_kb : kb0 + kb_per;
    };
    auto tile_coords = [&](int t, int& pm, int& pn) {
        constexpr int GROUP_M = @GROUP_M@;
        if (splits != 1) t -= quotient(t, base_tiles) * base_tiles;
        const int per_group = GROUP_M * grid_n;
        const int group = quotient(t, per_group);
        const int first = group * GROUP_M;
        const int rows = (grid_m - first < GROUP_M) ? (grid_m - first) : GROUP_M;
        const int in_group = t - group * per_group;
        pn = quotient(in_group, rows);
        pm = first + in_group - pn * rows;
    };

    if (num_kb > 0) {
        if (warp == 0 && lane == 0) {
            // ---------------- TMA producer ----------------
            unsigned it = 0;
            for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x) {
                int pm, pn, split, kb0, kb1;
                tile_coords(t, pm, pn);
                k_range(t, split, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const unsigned s = it % STAGES, phase = (it / STAGES) & 1u;
                    if (!mtb_mbar_wait(mtb_smem(&bar_empty[s]), phase ^ 1u, abort_flag, status, 0x10u + s)) break;
                    const unsigned full = mtb_smem(&bar_full[s]);
                    const unsigned a_dst = tiles_base + s * STAGE_BYTES;
                    const unsigned b_dst = a_dst + A_BYTES;
                    mtb_mbar_expect_tx(full, STAGE_BYTES);
                    if (A_MMAJOR) {
                        #pragma unroll
                        for (int j = 0; j < A_ROWS / AE; ++j)
                            mtb_tma_load_2d(a_dst + j * (BK * 128), &map_a, full, pm * BM + j * AE, kb * BK);
                    } else {
                        #pragma unroll
                        for (int j = 0; j < BK / AE; ++j)
                            mtb_tma_load_2d(a_dst + j * (A_ROWS * 128), &map_a, full, kb * BK + j * AE, pm * BM);
                    }
                    if (B_KMAJOR) {
                        #pragma unroll
                        for (int j = 0; j < BK / AE; ++j)
                            mtb_tma_load_2d(b_dst + j * (BN * 128), &map_b, full, kb * BK + j * AE, pn * BN);
                    } else {
                        #pragma unroll
                        for (int j = 0; j < BN / AE; ++j)
                            mtb_tma_load_2d(b_dst + j * (BK * 128), &map_b, full, pn * BN + j * AE, kb * BK);
                    }
                }
            }
        } else if (warp == 1 && lane == 0) {
            // ---------------- MMA issuer ----------------
            unsigned it = 0, local_tile = 0;
            for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x, ++local_tile) {
                const unsigned acc = local_tile & 1u, acc_phase = (local_tile >> 1) & 1u;
                if (!mtb_mbar_wait(mtb_smem(&bar_acc_empty[acc]), acc_phase ^ 1u, abort_flag, status, 0x20u + acc)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned d_tmem = tmem_base + acc * BN;
                bool ok = true;
                int split, kb0, kb1;
                k_range(t, split, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const unsigned s = it % STAGES, phase = (it / STAGES) & 1u;
                    if (!mtb_mbar_wait(mtb_smem(&bar_full[s]), phase, abort_flag, status, 0x30u + s)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned a_src = tiles_base + s * STAGE_BYTES;
                    const unsigned b_src = a_src + A_BYTES;
                    #pragma unroll
                    for (int k = 0; k < BK / UK; ++k) {
                        // A, K-major: UK k-elements = 32 bytes inside the 128-byte swizzle atom
                        const unsigned long long a_desc = !A_MMAJOR
                            ? mtb_desc(a_src + (k / 4) * (A_ROWS * 128) + (k % 4) * 32, 16, 1024)
                            : EB == 4
                            ? mtb_desc(a_src + k * 1024, BK * 128, 512, 1ull)
                            : mtb_desc(a_src + k * (UK / 8) * 1024, BK * 128, 1024);
                        // B, N-major: 2-byte elements are swizzled in 16-byte chunks over groups of
                        // 8 k-rows (1024 bytes), 16 k-rows per instruction; 4-byte elements only in
                        // 32-byte chunks over groups of 4 k-rows (512 bytes), 8 k-rows per
                        // instruction.  128-byte column sub-tiles are BK*128 bytes apart.
                        const unsigned long long b_desc = B_KMAJOR
                            ? mtb_desc(b_src + (k / 4) * (BN * 128) + (k % 4) * 32, 16, 1024)
                            : EB == 4
                            ? mtb_desc(b_src + k * 1024, BK * 128, 512, 1ull)
                            : mtb_desc(b_src + k * (UK / 8) * 1024, BK * 128, 1024);
                        mtb_umma_bf16(d_tmem, a_desc, b_desc, IDESC, (kb != kb0 || k != 0) ? 1u : 0u);
                    }
                    mtb_umma_commit(mtb_smem(&bar_empty[s]));      // stage free once these MMAs retire
                }
                if (!ok) break;
                mtb_umma_commit(mtb_smem(&bar_acc_full[acc]));     // accumulator complete
            }
        }
    }
    if (warp >= 2) {
        // ---------------- epilogue: TMEM -> registers -> global ----------------
        const int quad = warp & 3;                      // TMEM lane quadrant this warp may read
        unsigned local_tile = 0;
        for (int t = blockIdx.x; t < num_tiles && !*abort_flag; t += gridDim.x, ++local_tile) {
            int pm, pn, split, kb0, kb1;
            tile_coords(t, pm, pn);
            k_range(t, split, kb0, kb1);
            (void)split;
            const unsigned acc = local_tile & 1u, acc_phase = (local_tile >> 1) & 1u;
            if (num_kb > 0) {
                // the whole warp leaves together: tcgen05.ld below is warp-collective
                // one lane polls the barrier, the other 31 sleep at the shuffle; every lane then
                // makes its own (immediately successful) wait so that each of them has observed
                // the phase before it reads the accumulator
                unsigned ready = 1u;
                if (lane == 0) ready = mtb_mbar_wait(mtb_smem(&bar_acc_full[acc]), acc_phase, abort_flag, status, 0x40u + acc) ? 1u : 0u;
                ready = __shfl_sync(0xffffffffu, ready, 0);
                if (!ready) break;
                if (lane != 0) mtb_mbar_wait(mtb_smem(&bar_acc_full[acc]), acc_phase, abort_flag, status, 0x40u + acc);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            constexpr int MH = 1, h = 0;                // one 128-row half per CTA in this variant
@EPILOGUE_TILE@
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    // ---------------- teardown ----------------
    if (*abort_flag) {
        // let copies that are still in flight land before shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) { }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}
'''


def _c_type(param: Param) -> str:
    if isinstance(param.ty, PointerType):
        return {"bf16": "unsigned short*", "f16": "unsigned short*", "f32": "float*",
                "f8e4m3": "unsigned char*", "f8e5m2": "unsigned char*"}[param.ty.element.name]
    return "int" if param.ty == I32 else "float"


OUT_STAGING_BYTES = 4 * 2 * 32 * 32 * 4     # 4 epilogue warps x 2 boxes of 32x32 fp32


def choose_stages(bm: int, bn: int, bk: int, wanted: int | None, smem_limit: int = 227 * 1024,
                  elem_bytes: int = 2) -> int:
    stage = (bm * bk + bk * bn) * elem_bytes
    most = (smem_limit - 2048 - OUT_STAGING_BYTES) // stage
    stages = min(wanted or 8, most)
    if stages < 2:
        raise TypeError(f"tl.dot tile {bm}x{bn}x{bk} does not fit two pipeline stages in shared memory")
    return stages


_EPILOGUE_TILE = r"""            const int row_base = @ROW_BASE@;
            const int row = row_base + lane;
            constexpr bool OUT_BF16 = @OUT_BF16@;             // a 16-bit C: bf16 or fp16, rounded to nearest even
            constexpr bool C_TRANSPOSED = @C_TRANSPOSED@;     // element (row, col) is stored at col * ldc + row
            constexpr int BOX_COLS = OUT_BF16 ? 64 : 32;      // every staged row is 128 bytes of C
            const bool vec_ok = ((ldc & 3) == 0) && ((reinterpret_cast<unsigned long long>(@C@) & 15ull) == 0ull);
            const unsigned my_out = out_base + (unsigned)(warp - 2) * (2 * OUT_BYTES);
            #pragma unroll 1
            for (int box_index = 0; box_index < BN / BOX_COLS; ++box_index) {
                unsigned w[32];                               // this thread's row of the staging box
                #pragma unroll
                for (int half = 0; half < BOX_COLS / 32; ++half) {
                    const int chunk = box_index * (BOX_COLS / 32) + half;
                    unsigned v[32];
                    if (num_kb > 0) {
                        mtb_tmem_ld32(tmem_base + (acc * MH + h) * BN + ((unsigned)(quad * 32) << 16) + chunk * 32, v);
                    } else {
                        #pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = 0u;
                    }
                    if (num_kb > 0 && chunk == BN / 32 - 1) {
                        // accumulator fully read: hand it back before the stores drain
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        @RELEASE@
                    }
                    const int col0 = pn * BN + chunk * 32;   // first column of these 32 values
                    (void)col0;
@EPILOGUE@
                    if (OUT_BF16) {
                        #pragma unroll
                        for (int i = 0; i < 16; ++i)          // element 2i in the low half-word
                            asm("cvt.rn.@OUT_HALF@x2.f32 %0, %1, %2;" : "=r"(w[half * 16 + i])
                                : "f"(__uint_as_float(v[2 * i + 1])), "f"(__uint_as_float(v[2 * i])));
                    } else {
                        #pragma unroll
                        for (int i = 0; i < 32; ++i) w[i] = v[i];
                    }
                }
                const int box_col0 = pn * BN + box_index * BOX_COLS;
                if (n_dst > 0) {
                    // registers -> 128B-swizzled staging box -> TMA store (clipped at the
                    // matrix edge by the tensor map) to this GPU's C and to every peer's
                    const unsigned box = my_out + (unsigned)(box_index & 1) * OUT_BYTES;
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    __syncwarp();
                    if (C_TRANSPOSED) {
                        // the box holds the transpose: box row i = column box_col0 + i of the tile,
                        // 32 consecutive rows of it (one per lane) side by side, so every store
                        // instruction fills one whole 128-byte box row
                        #pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const unsigned dst = box + (unsigned)i * 128u
                                               + (unsigned)((((lane >> 2) ^ (i & 7)) << 4) | ((lane & 3) << 2));
                            asm volatile("st.shared.b32 [%0], %1;" :: "r"(dst), "r"(w[i]) : "memory");
                        }
                    } else {
                        #pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const unsigned dst = box + (unsigned)lane * 128u + (unsigned)((j ^ (lane & 7)) * 16);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                         :: "r"(dst), "r"(w[4 * j]), "r"(w[4 * j + 1]), "r"(w[4 * j + 2]), "r"(w[4 * j + 3])
                                         : "memory");
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        for (int d = 0; d < n_dst; ++d) {
                            if (C_TRANSPOSED) mtb_tma_store_2d(&maps_c.m[d], box, row_base, box_col0);
                            else mtb_tma_store_2d(&maps_c.m[d], box, box_col0, row_base);
                        }
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                } else if (C_TRANSPOSED) {
                    if (row < m_rows) {
                        float* out = reinterpret_cast<float*>(@C@);
                        #pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (box_col0 + i < n_cols)
                                out[(long long)(box_col0 + i) * ldc + row] = __uint_as_float(w[i]);
                    }
                } else if (row < m_rows) {
                    if (OUT_BF16) {
                        unsigned short* out_row = reinterpret_cast<unsigned short*>(@C@) + (long long)row * ldc;
                        #pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (box_col0 + 2 * i < n_cols) out_row[box_col0 + 2 * i] = (unsigned short)(w[i] & 0xffffu);
                            if (box_col0 + 2 * i + 1 < n_cols) out_row[box_col0 + 2 * i + 1] = (unsigned short)(w[i] >> 16);
                        }
                    } else {
                        float* out_row = reinterpret_cast<float*>(@C@) + (long long)row * ldc;
                        #pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            const int col = box_col0 + i;
                            if (vec_ok && col + 3 < n_cols) {
                                *reinterpret_cast<float4*>(out_row + col) = make_float4(
                                    __uint_as_float(w[i]), __uint_as_float(w[i + 1]),
                                    __uint_as_float(w[i + 2]), __uint_as_float(w[i + 3]));
                            } else {
                                #pragma unroll
                                for (int e = 0; e < 4; ++e)
                                    if (col + e < n_cols) out_row[col + e] = __uint_as_float(w[i + e]);
                            }
                        }
                    }
                }
            }
"""


def _epilogue_text(statements: tuple[str, ...]) -> str:
    if not statements:
        return ""
    pad = " " * 28
    body = "\n".join(pad + line for line in statements)
    return (
        "                    #pragma unroll\n"
        "                    for (int i = 0; i < 32; ++i) {\n"
        "                        const int col = col0 + i;\n"
        "                        float acc = __uint_as_float(v[i]);\n"
        "                        {\n" + body + "\n                        }\n"
        "                        v[i] = __float_as_uint(acc);\n"
        "                    }"
    )


_OPERAND_BYTES = {"bf16": 2, "f16": 2, "tf32": 4, "f8e4m3": 1, "f8e5m2": 1}

# The second kernel of a split-K launch: adds the units' partial sums in the order of the splits
# (so the result does not depend on which unit finished first), applies the kernel's epilogue
# and stores C.  One thread per four consecutive columns of a row.
_SPLIT_REDUCE = r'''
// x.to(tl.float16) / x.to(tl.bfloat16) in a fused epilogue: the value rounded to that precision
static __device__ __forceinline__ __attribute__((unused)) float mtb_round_f16(float f) {
    unsigned short h;
    asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f));
    asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h));
    return f;
}
static __device__ __forceinline__ __attribute__((unused)) float mtb_round_bf16(float f) {
    unsigned short h;
    asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(f));
    return __uint_as_float(((unsigned)h) << 16);
}
// an fp16 element of an epilogue vector or tile, widened
static __device__ __forceinline__ __attribute__((unused)) float mtb_half_bits_to_float(unsigned short h) {
    float f;
    asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h));
    return f;
}

extern "C" __global__ __launch_bounds__(256)
void @NAME@(@SIGNATURE@, const float* __restrict__ mtb_partial, int splits, long long split_stride,
            int partial_ld, int m_rows, int n_cols, int ldc) {
    constexpr bool OUT_BF16 = @OUT_BF16@;
    constexpr bool C_TRANSPOSED = @C_TRANSPOSED@;
    const int row = blockIdx.x;
    const int col0 = (blockIdx.y * 256 + threadIdx.x) * 4;
    if (row >= m_rows || col0 >= n_cols) return;
    const float* src = mtb_partial + (long long)row * partial_ld + col0;
    float4 sum = *reinterpret_cast<const float4*>(src);
    for (int s = 1; s < splits; ++s) {
        const float4 next = *reinterpret_cast<const float4*>(src + s * split_stride);
        sum.x += next.x; sum.y += next.y; sum.z += next.z; sum.w += next.w;
    }
    float v[4] = {sum.x, sum.y, sum.z, sum.w};
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int col = col0 + i;
        float acc = v[i];
        {
@EPILOGUE@
        }
        v[i] = acc;
        if (col < n_cols) {
            const long long at = C_TRANSPOSED ? (long long)col * ldc + row : (long long)row * ldc + col;
            if (OUT_BF16) {
                unsigned short bits;
                asm("cvt.rn.@OUT_HALF@.f32 %0, %1;" : "=h"(bits) : "f"(acc));
                reinterpret_cast<unsigned short*>(@C@)[at] = bits;
            } else {
                reinterpret_cast<float*>(@C@)[at] = acc;
            }
        }
    }
}
'''


def generate_gemm(kernel_name: str, match: GemmMatch, params: list[Param], codegen) -> Any:
    from . import dot_codegen_pair as pair
    from .cuda_codegen import KernelArtifact, LaunchPlan

    # default: pair two CTAs (256 x BN tile) whenever B can be split in 64-column boxes
    skinny = getattr(codegen, "a_rows", None) is not None
    a_rows = getattr(codegen, "a_rows", None) or 128
    if skinny:
        # the skinny variant: the launch covers at most a_rows rows, so only those rows of A are
        # fetched, the tile is narrowed to one 128-byte column box (many CTAs, each streaming its
        # own slice of B) and the space saved goes into pipeline stages
        if a_rows % 8 or not 8 <= a_rows <= 128:
            raise ValueError(f"a_rows must be a multiple of 8 up to 128, got {a_rows}")
        if (getattr(codegen, "cta_group", None) or 1) != 1 or match.bm == 256:
            raise TypeError("a_rows applies to the single-CTA kernel (cta_group=1, BM=128)")
        if match.a_transposed:
            raise TypeError("a_rows applies to A stored [M, K]: a transposed A is fetched 64 rows at a time")
        import dataclasses

        atom = 128 // _OPERAND_BYTES[match.operand]
        # deep k-blocks: with so little arithmetic per block the producer/consumer hand-over
        # is what each block costs, so there should be few of them
        match = dataclasses.replace(match, bn=max(64, atom), bk=(4 if a_rows <= 64 else 2) * atom,
                                    program_tile=match.program_tile or (match.bm, match.bn))
    tile_n = getattr(codegen, "tile_n", None)
    if tile_n is not None:
        # the kernel's own tile width: the programs' tiles only say which part of C a launch
        # covers, so a problem with few tiles may be cut into narrower ones that fill the GPU
        import dataclasses

        atom = 128 // _OPERAND_BYTES[match.operand]
        if tile_n not in (64, 128, 256) or tile_n % max(64, atom):
            raise ValueError(f"tile_n must be 64, 128 or 256 and a multiple of {max(64, atom)}, got {tile_n}")
        if match.bm != 128:
            raise TypeError("tile_n applies to kernels with a 128-row tile")
        bk = match.bk
        if skinny:          # keep a stage near 48 KiB so that several fit
            bk = atom * max(1, min(bk // atom, 48 * 1024 // ((a_rows + tile_n) * _OPERAND_BYTES[match.operand]) // atom))
        match = dataclasses.replace(match, bn=tile_n, bk=bk, program_tile=match.program_tile or (match.bm, match.bn))
    split_k = getattr(codegen, "split_k", None) or 1
    if split_k < 1:
        raise ValueError(f"split_k must be a positive number of splits, got {split_k}")
    if split_k > 1 and ((getattr(codegen, "cta_group", None) or 1) != 1 or match.bm != 128):
        raise TypeError("split_k applies to the single-CTA kernel (cta_group=1, 128-row tiles)")
    pair_columns = max(128, 2 * (128 // _OPERAND_BYTES[match.operand]))   # two 128-byte column boxes
    cta_group = 1 if skinny or split_k > 1 else (
        getattr(codegen, "cta_group", None) or (2 if match.bn % pair_columns == 0 else 1))
    if cta_group not in (1, 2):
        raise ValueError(f"cta_group must be 1 or 2, got {cta_group}")
    if match.bm == 256 and cta_group != 2:
        raise TypeError("a 256-row tl.dot tile is computed by a CTA pair: cta_group must be 2")
    if cta_group == 2 and match.bn % pair_columns:
        raise TypeError(f"cta_group=2 splits B between two CTAs in 128-byte column boxes: "
                        f"BN must be a multiple of {pair_columns}")
    # rows of the tile one CTA holds in TMEM: 128, or 256 as two 128-row halves that share B
    # (the default where such a tile exists: a CTA pair with BN = 256 and a 128-row program tile)
    cta_rows = getattr(codegen, "cta_rows", None) or (
        256 if cta_group == 2 and match.bn == 256 and match.bm == 128 else 128)
    if cta_rows not in (128, 256):
        raise ValueError(f"cta_rows must be 128 or 256, got {cta_rows}")
    if cta_rows == 256 and cta_group != 2:
        raise TypeError("cta_rows=256 is a variant of the CTA-pair kernel: cta_group must be 2")
    halves = cta_rows // 128
    if halves * match.bn > 512:
        raise TypeError(f"a {cta_rows} x {match.bn} fp32 accumulator does not fit the 512 TMEM columns")
    accumulators = 2 if 2 * halves * match.bn <= 512 else 1
    tmem_cols = 32
    while tmem_cols < accumulators * halves * match.bn:
        tmem_cols *= 2
    elem_bytes = _OPERAND_BYTES[match.operand]
    if cta_group == 2:
        stage = pair.pair_stage_bytes(cta_rows, match.bn, match.bk, elem_bytes)
        most = (227 * 1024 - 2048 - pair.PAIR_OUT_STAGING_BYTES) // stage
        stages = min(codegen.num_stages or 8, most)
        if stages < 2:
            raise TypeError("tl.dot tile does not fit two pipeline stages in shared memory")
    else:
        stage = (a_rows * match.bk + match.bk * match.bn) * elem_bytes
        stages = choose_stages(a_rows, match.bn, match.bk, codegen.num_stages or (16 if skinny else None),
                               elem_bytes=elem_bytes)
    release = ("if (lane == 0) mtb_mbar_arrive(mtb_smem(&bar_acc_empty[acc * MH + h]));" if cta_group == 1 else
               "if (lane == 0) mtb_mbar_arrive_cluster(mtb_mapa(mtb_smem(&bar_acc_empty[acc * MH + h]), 0u));")
    row_base = ("split * split_rows + pm * BM + quad * 32" if cta_group == 1
                else "((pm * 2 + (int)rank) * MH + h) * BM + quad * 32")
    splitting = split_k > 1         # the GEMM kernel then stores raw fp32 partial sums, row-major
    substitutions = {
        "EPILOGUE_TILE": _EPILOGUE_TILE.replace("@RELEASE@", release).replace("@ROW_BASE@", row_base),
        "OUT_BF16": "true" if match.out in ("bf16", "f16") and not splitting else "false",
        "OUT_HALF": "f16" if match.out == "f16" else "bf16",
        "C_TRANSPOSED": "true" if match.c_transposed and not splitting else "false",
        "B_KMAJOR": "true" if match.b_transposed else "false",
        "A_MMAJOR": "true" if match.a_transposed else "false",
        "SPLIT_PARAMS": "int splits, int kb_per, int split_rows, " if splitting else "",
        "SPLIT_DECLS": "" if splitting else "constexpr int splits = 1, kb_per = 1 << 30, split_rows = 0;",
        "NAME": kernel_name,
        "SIGNATURE": ", ".join(f"{_c_type(p)} {p.name}" for p in params),
        "BM": 128, "BN": match.bn, "BK": match.bk, "STAGES": stages, "A_ROWS": a_rows,
        "MH": halves, "ACCS": accumulators,
        "TMEM_COLS": tmem_cols, "GROUP_M": getattr(codegen, "group_m", None) or 16 // cta_group,
        "C": match.c.name,
        "EPILOGUE": "" if splitting else _epilogue_text(match.epilogue),
        "AB_FORMAT": {"f16": 0, "bf16": 1, "tf32": 2, "f8e4m3": 0, "f8e5m2": 1}[match.operand],
        "EB": elem_bytes,
    }
    kind = {"tf32": "tf32", "f8e4m3": "f8f6f4", "f8e5m2": "f8f6f4"}.get(match.operand, "f16")
    prelude = f'#define MTB_WAIT_LIMIT {WAIT_LIMIT_CYCLES}ll\n#define MTB_MMA_KIND "{kind}"\n' + _PRELUDE
    if cta_group == 2:
        src = pair.pair_source(prelude, substitutions)
    else:
        text = _KERNEL
        for key, value in substitutions.items():
            text = text.replace(f"@{key}@", str(value))
        src = prelude + text
    plan = LaunchPlan(
        kernel_name=kernel_name,
        threads=192,
        dynamic_smem=stages * stage + OUT_STAGING_BYTES + 1024,
        kind="tcgen05",
    )
    plan.notes["gemm"] = match
    plan.notes["stages"] = stages
    plan.notes["cta_group"] = cta_group
    plan.notes["a_rows"] = a_rows
    plan.notes["cta_rows"] = cta_rows
    plan.notes["skinny"] = skinny
    plan.notes["split_k"] = split_k
    if splitting:
        reduce_name = kernel_name + "_add_splits"
        pad = " " * 12
        reduce_src = _SPLIT_REDUCE
        for key, value in {
            "NAME": reduce_name, "SIGNATURE": substitutions["SIGNATURE"], "C": match.c.name,
            "OUT_BF16": "true" if match.out in ("bf16", "f16") else "false",
            "OUT_HALF": "f16" if match.out == "f16" else "bf16",
            "C_TRANSPOSED": "true" if match.c_transposed else "false",
            "EPILOGUE": "\n".join(pad + line for line in match.epilogue),
        }.items():
            reduce_src = reduce_src.replace(f"@{key}@", str(value))
        plan.notes["add_splits"] = (reduce_src, reduce_name)
    plan.cluster = (cta_group, 1, 1)
    return KernelArtifact(src, plan)


# --------------------------------------------------------------------------- launch-time work

_status_words: dict[int, int] = {}


def status_word(runtime) -> int:
    """One zero-initialised 32-bit status word per device, allocated on first use."""
    device = runtime.current_device()
    if device not in _status_words:
        ptr = runtime.mem_alloc(256)
        runtime.memset_u32(ptr, 0, 64)
        runtime.synchronize()
        _status_words[device] = ptr
    return _status_words[device]


def check_status(stream: int = 0) -> None:
    """Synchronise ``stream`` and raise if a tcgen05 kernel reported a timed-out wait."""
    from . import runtime

    device = runtime.current_device()
    if device in _status_words:
        try:
            runtime.status_check(_status_words[device], stream)
        except runtime.RuntimeLibraryError:
            # reported once: later, healthy launches must not keep failing on an old code
            runtime.memset_u32(_status_words[device], 0, 1, stream)
            runtime.stream_synchronize(stream)
            raise


def _resolve(symbol: str | None, runtime_args, names, default: int) -> int:
    if symbol is None:
        return default
    if symbol.startswith("#"):
        return int(symbol[1:])
    return int(runtime_args[names.index(symbol[2:])])


class GemmLaunchError(ValueError):
    pass


_tensormap_cache: dict[tuple, Any] = {}


_tile_rectangles: dict[tuple, tuple[int, int]] = {}


def _c_quotient(a, b):
    """Integer division that truncates toward zero, as the generated C does."""
    import numpy as np

    return np.sign(a) * np.sign(b) * (np.abs(a) // np.abs(b))


def _evaluate_tile_map(tile_map: TileMap, grid: tuple[int, int, int], scalars: dict[str, int]) -> tuple[int, int]:
    """Runs the kernel's program -> tile arithmetic for every program of ``grid`` (NumPy, on the
    host) and returns (tile rows, tile columns) of the rectangle they cover, or raises
    GemmLaunchError when the programs that do any work do not visit every tile of a rectangle
    exactly once — then the launch is no dense GEMM and the tensor-core kernel must not stand in."""
    import numpy as np

    total = grid[0] * grid[1] * grid[2]
    if total > 1 << 22:
        raise GemmLaunchError(f"{total} programs: too many to check the program -> tile map")
    ids = np.arange(total, dtype=np.int64)
    env = {"pid0": ids % grid[0], "pid1": (ids // grid[0]) % grid[1], "pid2": ids // (grid[0] * grid[1])}
    opaque = dict(tile_map.opaque)
    undefined = np.zeros(total, dtype=bool)          # programs that divide by zero on the way

    def lookup(symbol: str):
        if symbol not in env:
            if symbol.startswith("p:"):
                if symbol[2:] not in scalars:
                    raise GemmLaunchError(f"the program -> tile map reads {symbol[2:]}, which is not an integer argument")
                env[symbol] = np.int64(scalars[symbol[2:]])
            else:
                code, lhs, rhs = opaque[symbol]
                a, b = value(lhs), value(rhs)
                if code in ("div", "rem"):
                    zero = np.broadcast_to(b == 0, (total,))
                    undefined[:] |= zero
                    b = np.where(b == 0, 1, b)
                    quotient = _c_quotient(a, b)
                    env[symbol] = quotient if code == "div" else a - quotient * b
                else:
                    env[symbol] = np.minimum(a, b) if code == "minimum" else np.maximum(a, b)
        return env[symbol]

    def value(poly: Poly):
        out = np.int64(0)
        for monomial, coefficient in poly.terms.items():
            term = np.int64(coefficient)
            for symbol in monomial:
                term = term * lookup(symbol)
            out = out + term
        return out

    active = np.ones(total, dtype=bool)
    for guard in tile_map.guards:
        active &= np.broadcast_to(value(guard.lhs) < value(guard.rhs), (total,))
    rows = np.broadcast_to(value(tile_map.row_tile), (total,))[active]
    cols = np.broadcast_to(value(tile_map.col_tile), (total,))[active]
    if rows.size == 0:
        raise GemmLaunchError("no program of this grid does any work")
    if undefined[active].any():
        raise GemmLaunchError("a program divides by zero while locating its tile")
    tiles_m, tiles_n = int(rows.max()) + 1, int(cols.max()) + 1
    if rows.min() < 0 or cols.min() < 0 or rows.size != tiles_m * tiles_n \
            or np.unique(rows * tiles_n + cols).size != rows.size:
        raise GemmLaunchError("the programs of this grid do not visit every tile of a rectangle exactly once")
    return tiles_m, tiles_n


def launch_tiles(match: GemmMatch, launch_grid, runtime_args, names) -> tuple[int, int]:
    """(rows, columns) of the rectangle of program tiles a launch covers."""
    grid = tuple(int(d) for d in launch_grid) + (1,) * (3 - len(launch_grid))
    if match.tile_map is None:
        spare = ({0, 1, 2} - {match.axis_m, match.axis_n}).pop()
        if grid[spare] != 1:
            raise GemmLaunchError("tl.dot kernels use two grid axes; the third must be 1")
        return grid[match.axis_m], grid[match.axis_n]
    import numpy as np

    scalars = {name: int(value) for name, value in zip(names, runtime_args)
               if isinstance(value, (int, np.integer)) and not isinstance(value, bool)}
    key = (match.tile_map, grid, tuple(sorted(scalars.items())))
    if key not in _tile_rectangles:
        if len(_tile_rectangles) > 256:
            _tile_rectangles.clear()
        _tile_rectangles[key] = _evaluate_tile_map(match.tile_map, grid, scalars)
    return _tile_rectangles[key]


def launch_obstacle(plan, launch_grid, runtime_args, param_names) -> str | None:
    """Why this launch cannot take the TMA/tcgen05 kernel (None if it can): TMA wants
    16-byte aligned operands with row strides of whole 16-byte units, and the kernel maps
    programs to tiles over two grid axes.  The caller then uses the SIMT variant."""
    from . import arrays

    match: GemmMatch = plan.notes["gemm"]
    names = list(param_names)
    try:
        launch_tiles(match, launch_grid, runtime_args, names)
    except GemmLaunchError as error:
        return str(error)
    lda = _resolve(match.lda, runtime_args, names, 0)
    ldb = _resolve(match.ldb, runtime_args, names, 0)
    elem_bytes = _OPERAND_BYTES[match.operand]
    addresses = [arrays.describe(runtime_args[names.index(p.name)]).address or 0 for p in (match.a, match.b)]
    if (lda * elem_bytes) % 16 or (ldb * elem_bytes) % 16 or any(address % 16 for address in addresses):
        return ("the tcgen05 path needs 16-byte aligned operands whose row strides are "
                f"multiples of 16 bytes (lda={lda}, ldb={ldb}, {elem_bytes}-byte elements)")
    return None


def skinny_rows(plan, launch_grid, runtime_args, param_names) -> int | None:
    """16, 32, 64 or 128 when this launch covers at most that many rows of C (a skinny problem that
    streams B once: the variant that fetches only those rows of A is the better kernel), else None."""
    match: GemmMatch = plan.notes["gemm"]
    if plan.notes.get("skinny") or match.bm != 128 or match.tile_map is not None or match.c_transposed \
            or match.a_transposed:          # (a transposed A is fetched 64 rows at a time: no few-row form)
        return None
    names = list(param_names)
    grid = tuple(launch_grid) + (1,) * (3 - len(launch_grid))
    program_bm = (match.program_tile or (match.bm, match.bn))[0]
    covered = grid[match.axis_m] * program_bm
    rows = min(_resolve(match.m_extent, runtime_args, names, covered), covered)
    for bucket in (16, 32, 64, 128):
        if rows <= bucket:
            return bucket
    return None


def skinny_launch_options(plan, launch_grid, runtime_args, param_names) -> dict | None:
    """``skinny_options`` for one launch, or None when the launch is no skinny problem."""
    from . import runtime

    rows = skinny_rows(plan, launch_grid, runtime_args, param_names)
    if rows is None:
        return None
    match: GemmMatch = plan.notes["gemm"]
    names = list(param_names)
    grid = tuple(launch_grid) + (1,) * (3 - len(launch_grid))
    program_bn = (match.program_tile or (match.bm, match.bn))[1]
    covered = grid[match.axis_n] * program_bn
    cols = min(_resolve(match.n_extent, runtime_args, names, covered), covered)
    depth = _resolve(match.k_extent, runtime_args, names, 0)
    device = runtime.current_device()
    if device not in _sm_counts:
        _sm_counts[device] = runtime.device_info(device).sm_count
    return skinny_options(rows, cols, depth, 128 // _OPERAND_BYTES[match.operand], _sm_counts[device])


def skinny_options(rows: int, cols: int, depth: int, atom: int, sms: int) -> dict:
    """Code-generation options of the skinny variant for a launch of at most ``rows`` (a bucket: 16,
    32, 64 or 128) rows of C.  Such a launch streams B once, at best at the rate of HBM; what it
    adds is re-reading A through L2 once per column tile, and it needs about one unit of work per
    SM.  So: 128-column tiles (half the re-reads of 64-column ones) with as many units along K as
    fill the SMs, at least sixteen k-blocks each; 64-column tiles when K is too shallow to split
    and 128-column tiles would leave half of the SMs idle.  Measured (bf16, fp32 C, CUDA-graph
    replay): 128 x 8192 x 8192 33.7 -> 31.0 us, 128 x 4096 x 16384 57.4 -> 30.8 us,
    32 x 16384 x 4096 29.0 -> 25.2 us."""
    options: dict = {"a_rows": rows}
    if cols <= 64 or 128 % max(64, atom):
        return options
    tiles = -(-cols // 128)
    elem_bytes = 128 // atom
    bk = atom * max(1, min(4 if rows <= 64 else 2, 48 * 1024 // ((rows + 128) * elem_bytes) // atom))
    blocks = -(-depth // bk)
    splits = max(1, min(16, sms // tiles, blocks // 16))
    if rows <= 64 and splits < 4:
        # little of A to re-read: two or three units per tile gain less than the second launch costs
        # (16 x 8192 x 8192: 28.4 -> 27.8 us under graph replay, 30.0 -> 32.9 us launched from a stream)
        splits = 1
    if splits == 1 and 2 * tiles <= sms:
        return options
    options["tile_n"] = 128
    if splits > 1:
        options["split_k"] = splits
    return options


_sm_counts: dict[int, int] = {}


# A 512-row tile fills all of tensor memory with one accumulator, so part of its epilogue runs with
# the tensor cores idle; the 256-row tiling has two accumulators and hides the epilogue completely.
# The wide tile's saving in operand traffic grows with K while the exposed epilogue does not:
# measured on 8192 x 8192 and 32768 x 8192 outputs, bf16, the two tilings are level at K = 4096
# (1.46 vs 1.45 PFLOP/s), the narrow one is ahead below it (K = 1024: 1.17 vs 1.05) and the wide one
# above it (K = 8192: 1.53 vs 1.46).
WIDE_TILE_MIN_DEPTH = 4096


def prefers_narrow_tiles(plan, launch_grid, runtime_args, param_names) -> bool:
    """True when the 256-row tiling serves this launch better than the 512-row tiling the kernel was
    built with.  Two reasons: a shallow K (see WIDE_TILE_MIN_DEPTH), and fill — every CTA pair takes
    whole tiles, so a launch with few 512-row tiles (fewer than pairs, or a little more than a whole
    number of rounds) leaves part of the GPU idle, and halving the tile height can fill it."""
    from . import runtime

    if plan.notes.get("cta_rows", 128) != 256:
        return False
    match: GemmMatch = plan.notes["gemm"]
    names = list(param_names)
    try:
        tiles_m, tiles_n = launch_tiles(match, launch_grid, runtime_args, names)
    except GemmLaunchError:
        return False
    program_bm, program_bn = match.program_tile or (match.bm, match.bn)
    rows = min(_resolve(match.m_extent, runtime_args, names, tiles_m * program_bm), tiles_m * program_bm)
    cols = min(_resolve(match.n_extent, runtime_args, names, tiles_n * program_bn), tiles_n * program_bn)
    depth = _resolve(match.k_extent, runtime_args, names, 0)
    if 0 < depth < WIDE_TILE_MIN_DEPTH:
        return True
    device = runtime.current_device()
    if device not in _sm_counts:
        _sm_counts[device] = runtime.device_info(device).sm_count
    return narrow_tiles_fill_better(rows, cols, match.bn, max(1, _sm_counts[device] // 2))


def small_problem_variant(rows: int, cols: int, depth: int, bk: int, atom: int, sms: int) -> dict | None:
    """Code-generation options for a launch with too few tiles to fill the GPU with CTA pairs, or
    None to keep the pair kernel.

    The single-CTA kernel can cut such a problem into more units of work: narrower tiles
    (``tile_n``) and, where K is deep, several units per tile along K (``split_k``) whose partial
    sums a second kernel adds up.  The choice follows a model of the launch, in microseconds,
    fitted to measurements on a B200 (bf16; 1024^3 ... 512 x 512 x 16384): a fixed cost per launch
    (10 us for CTA pairs, 6 us for single CTAs), per round of units the k-blocks of one unit at
    0.3 us each (1.12 x that for single CTAs, which share no operand) plus filling the pipeline and
    draining the tile (2 us for 256 columns), and 4-8 us for the second kernel.
    Measured: 1024 x 1024 x 8192 43 -> 23 us with four splits, 512 x 512 x 16384 80 -> 22 us with
    eight, 1024^3 14.5 -> 10.5 us with 64-column tiles."""
    if depth <= 0 or rows <= 128:
        return None
    pairs = max(1, sms // 2)
    pair_tiles = -(-rows // 256) * -(-cols // 256)
    if pair_tiles > 2 * pairs:
        return None
    blocks = -(-depth // bk)
    per_block = 0.3 * bk / atom         # one 128-byte swizzle row of k per 0.3 us, whatever the element type
    best, best_time = None, 0.97 * (10.2 + -(-pair_tiles // pairs) * blocks * per_block)
    for tile_n in (256, 128, 64):
        if tile_n % max(64, atom):
            continue
        tiles = -(-rows // 128) * -(-cols // tile_n)
        for splits in (1, 2, 3, 4, 6, 8, 12, 16):
            if splits > 1 and blocks // splits < 4:
                break
            rounds = -(-tiles * splits // sms)
            time = (6.1 + rounds * (-(-blocks // splits) * per_block * 1.12 + 2.0 * tile_n / 256)
                    + (4.0 + 0.25 * splits if splits > 1 else 0.0))
            if time < best_time:
                best, best_time = {"cta_group": 1, "tile_n": tile_n, **({"split_k": splits} if splits > 1 else {})}, time
    return best


def prefers_small_problem_variant(plan, launch_grid, runtime_args, param_names) -> dict | None:
    """``small_problem_variant`` for one launch of a kernel compiled with the default options."""
    from . import runtime

    match: GemmMatch = plan.notes["gemm"]
    if plan.notes.get("cta_group") != 2 or match.bm != 128 or plan.notes.get("skinny"):
        return None
    names = list(param_names)
    try:
        tiles_m, tiles_n = launch_tiles(match, launch_grid, runtime_args, names)
    except GemmLaunchError:
        return None
    program_bm, program_bn = match.program_tile or (match.bm, match.bn)
    rows = min(_resolve(match.m_extent, runtime_args, names, tiles_m * program_bm), tiles_m * program_bm)
    cols = min(_resolve(match.n_extent, runtime_args, names, tiles_n * program_bn), tiles_n * program_bn)
    depth = _resolve(match.k_extent, runtime_args, names, 0)
    device = runtime.current_device()
    if device not in _sm_counts:
        _sm_counts[device] = runtime.device_info(device).sm_count
    return small_problem_variant(rows, cols, depth, match.bk, 128 // _OPERAND_BYTES[match.operand], _sm_counts[device])


def narrow_tiles_fill_better(rows: int, cols: int, bn: int, pairs: int) -> bool:
    """Whether 256-row pair tiles beat 512-row ones for a rows x cols output on ``pairs`` CTA pairs.

    Every pair takes whole tiles, one after the other, and a tile costs the same whether or not all
    of its rows exist; so the launch lasts (rounds of tiles) x (time of one tile), and per row a
    512-row tile is about 6 % cheaper (less operand traffic per flop)."""
    wide_rounds = -(-(-(-rows // 512) * -(-cols // bn)) // pairs)
    narrow_rounds = -(-(-(-rows // 256) * -(-cols // bn)) // pairs)
    return narrow_rounds * 256 < wide_rounds * 512 / 1.06


def prepare_launch(plan, runtime, info, launch_grid, runtime_args, param_names, peer_stores=None):
    """Returns (cuda_grid, extra_args): tensor maps, logical grid, extents, status.

    ``peer_stores`` maps the output parameter's name to a list of device addresses:
    every finished tile is written to each of them (this GPU's C and the same rows
    of every peer's C), which fuses the all-gather into the GEMM epilogue."""
    from . import arrays

    match: GemmMatch = plan.notes["gemm"]
    names = list(param_names)
    tiles_m, tiles_n = launch_tiles(match, launch_grid, runtime_args, names)
    # the part of C this launch covers: the programs' tiles, clipped by the masks' extents
    program_bm, program_bn = match.program_tile or (match.bm, match.bn)
    covered_rows = tiles_m * program_bm
    covered_cols = tiles_n * program_bn
    k_depth = _resolve(match.k_extent, runtime_args, names, 0)
    m_rows = min(_resolve(match.m_extent, runtime_args, names, covered_rows), covered_rows)
    n_cols = min(_resolve(match.n_extent, runtime_args, names, covered_cols), covered_cols)
    grid_m = max(1, -(-m_rows // 128))        # the kernel's own tiles: 128 rows per CTA, BN columns
    grid_n = max(1, -(-n_cols // match.bn))
    lda = _resolve(match.lda, runtime_args, names, 0)
    ldb = _resolve(match.ldb, runtime_args, names, 0)
    ldc = _resolve(match.ldc, runtime_args, names, 0)
    a_addr = arrays.describe(runtime_args[names.index(match.a.name)]).address
    b_addr = arrays.describe(runtime_args[names.index(match.b.name)]).address
    elem_bytes = _OPERAND_BYTES[match.operand]
    if (lda * elem_bytes) % 16 or (ldb * elem_bytes) % 16 or a_addr % 16 or b_addr % 16:
        raise GemmLaunchError(
            "the tcgen05 path needs 16-byte aligned operands whose row strides are "
            f"multiples of 16 bytes (lda={lda}, ldb={ldb}, {elem_bytes}-byte elements)"
        )
    a_rows = plan.notes.get("a_rows", 128)
    if m_rows > a_rows and plan.notes.get("skinny"):
        raise GemmLaunchError(f"this variant fetches {a_rows} rows of A; the launch covers {m_rows}")
    cta_rows = plan.notes.get("cta_rows", 128)
    box_rows = a_rows if plan.notes.get("skinny") else cta_rows      # rows of A one TMA box brings in
    pair = plan.notes.get("cta_group", 1) == 2
    key = (a_addr, b_addr, m_rows, n_cols, k_depth, lda, ldb, match.bm, match.bn, match.bk, match.operand, box_rows,
           match.b_transposed, pair, match.a_transposed)
    maps = _tensormap_cache.get(key)
    if maps is None:
        bf16, atom = match.operand == "bf16", 128 // elem_bytes
        if match.a_transposed:
            # A as [K, M]: the MN-major operand, boxes of [BK rows of k][128 bytes of rows of the tile]
            map_a = runtime.encode_tensormap_2d(
                a_addr, m_rows, k_depth, lda * elem_bytes, atom, match.bk, elem_bytes=elem_bytes, is_bf16=bf16,
                swizzle=runtime.SWIZZLE_128B_ATOM_32B if elem_bytes == 4 else runtime.SWIZZLE_128B)
        else:
            map_a = runtime.encode_tensormap_2d(a_addr, k_depth, m_rows, lda * elem_bytes, atom, box_rows,
                                                elem_bytes=elem_bytes, is_bf16=bf16)
        if match.b_transposed:
            # B as [N, K]: K-major like A; one box brings in the tile's columns (half of them per
            # CTA of a pair) as rows of 128 bytes of k
            map_b = runtime.encode_tensormap_2d(
                b_addr, k_depth, n_cols, ldb * elem_bytes, atom, match.bn // 2 if pair else match.bn,
                elem_bytes=elem_bytes, is_bf16=bf16)
        else:
            map_b = runtime.encode_tensormap_2d(
                b_addr, n_cols, k_depth, ldb * elem_bytes, atom, match.bk, elem_bytes=elem_bytes, is_bf16=bf16,
                # N-major B of 4-byte elements is swizzled in 32-byte chunks (its only legal form)
                swizzle=runtime.SWIZZLE_128B_ATOM_32B if elem_bytes == 4 else runtime.SWIZZLE_128B)
        if len(_tensormap_cache) > 64:
            _tensormap_cache.clear()
        maps = _tensormap_cache[key] = (map_a, map_b)
    c_addr = arrays.describe(runtime_args[names.index(match.c.name)]).address
    if plan.notes.get("split_k", 1) > 1:
        return _prepare_split_launch(plan, runtime, info, runtime_args, maps, grid_m, grid_n, m_rows, n_cols,
                                     k_depth, ldc, peer_stores)
    destinations = list((peer_stores or {}).get(match.c.name, [c_addr]))
    if len(destinations) > 8:
        raise GemmLaunchError("at most 8 destinations per output tile")
    maps_c = runtime.aligned_struct(runtime.TensorMaps8)
    n_dst = 0
    out_bytes = 2 if match.out in ("bf16", "f16") else 4
    if (ldc * out_bytes) % 16 == 0 and all(addr % 16 == 0 for addr in destinations):
        # C as the store sees it: [m_rows][n_cols] with rows ldc apart, or its transpose
        inner, outer = (m_rows, n_cols) if match.c_transposed else (n_cols, m_rows)
        for index, addr in enumerate(destinations):
            runtime.encode_tensormap_2d(
                addr, inner, outer, ldc * out_bytes, 128 // out_bytes, 32, elem_bytes=out_bytes,
                is_float=True, is_bf16=match.out == "bf16", out=ctypes.addressof(maps_c.m[index]))
        n_dst = len(destinations)
    elif peer_stores:
        raise GemmLaunchError("peer stores need a 16-byte aligned C whose row stride is a multiple of 16 bytes")
    if plan.notes.get("cta_group", 1) == 2:
        tile_rows = 2 * (cta_rows // 128)          # 128-row tiles of C in one pair tile
        pairs = max(1, min(-(-grid_m // tile_rows) * grid_n, info.sm_count // 2))
        ctas = 2 * pairs
    else:
        ctas = max(1, min(grid_m * grid_n, info.sm_count))
    extra = [
        maps[0], maps[1], maps_c, ctypes.c_int32(n_dst),
        ctypes.c_int32(grid_m), ctypes.c_int32(grid_n), ctypes.c_int32(m_rows),
        ctypes.c_int32(n_cols), ctypes.c_int32(k_depth), ctypes.c_int32(ldc),
        ctypes.c_uint64(status_word(runtime)),
    ]
    return (ctas,), extra, None


def _prepare_split_launch(plan, runtime, info, runtime_args, maps, grid_m, grid_n, m_rows, n_cols, k_depth, ldc,
                          peer_stores):
    """The two launches of a split-K GEMM: the units' kernel, which stores partial sums into a
    workspace of [splits][grid_m * 128][grid_n * BN] floats owned by this prepared launch, and the
    kernel that adds them up.  Launch objects made from one call share the workspace: they must not
    run at the same time on different streams."""
    from . import device

    if peer_stores:
        raise GemmLaunchError("peer stores are written by the GEMM's epilogue; a split-K launch has none")
    match: GemmMatch = plan.notes["gemm"]
    num_kb = -(-k_depth // match.bk)
    kb_per = max(1, -(-num_kb // plan.notes["split_k"]))
    splits = max(1, -(-num_kb // kb_per))           # every split has at least one k-block
    split_rows, partial_ld = grid_m * 128, grid_n * match.bn
    workspace = device.DeviceArray((splits * split_rows, partial_ld))
    maps_c = runtime.aligned_struct(runtime.TensorMaps8)
    runtime.encode_tensormap_2d(workspace.ptr, partial_ld, splits * split_rows, partial_ld * 4, 32, 32,
                                elem_bytes=4, is_float=True, is_bf16=False, out=ctypes.addressof(maps_c.m[0]))
    ctas = max(1, min(grid_m * grid_n * splits, info.sm_count))
    extra = [
        maps[0], maps[1], maps_c, ctypes.c_int32(1),
        ctypes.c_int32(grid_m), ctypes.c_int32(grid_n), ctypes.c_int32(splits * split_rows),
        ctypes.c_int32(partial_ld), ctypes.c_int32(k_depth), ctypes.c_int32(partial_ld),
        ctypes.c_int32(splits), ctypes.c_int32(kb_per), ctypes.c_int32(split_rows),
        ctypes.c_uint64(status_word(runtime)),
    ]
    source, name = plan.notes["add_splits"]
    follow_up = {
        "src": source, "name": name, "threads": 256,
        "grid": (m_rows, -(-n_cols // 1024)),
        "args": [ctypes.c_uint64(workspace.ptr), ctypes.c_int32(splits),
                 ctypes.c_int64(split_rows * partial_ld), ctypes.c_int32(partial_ld),
                 ctypes.c_int32(m_rows), ctypes.c_int32(n_cols), ctypes.c_int32(ldc)],
        "keepalive": workspace,
    }
    return (ctas,), extra, follow_up


# --------------------------------------------------------------------------- build / smoke probes


def compile_probe() -> None:
    """NVRTC-compile the GEMM kernel for the benchmark tile (needs no GPU)."""
    from . import runtime
    from .cuda_utils import NVRTC_OPTIONS
    from .types import PTR_BF16, PTR_F32

    params = [Param("a", PTR_BF16), Param("b", PTR_BF16), Param("c", PTR_F32),
              Param("M", I32), Param("N", I32), Param("K", I32)]
    match = GemmMatch(params[0], params[1], params[2], 128, 256, 64, 0, 1,
                      "p:K", "p:N", "p:N", "p:K", "p:M", "p:N")

    class _Options:
        num_stages = None

    artifact = generate_gemm("mtb_gemm_probe", match, params, _Options())
    runtime.Module(artifact.src, "mtb_gemm_probe", NVRTC_OPTIONS)
