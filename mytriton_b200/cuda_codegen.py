"""SSA -> CUDA C++ for sm_100a.

The entry point keeps the reference's shape — ``SSACUDACodegen().generate(
kernel_name, ssa_ops, params) -> str`` (``src/mytriton/cuda_codegen.py:436-472``)
— and so do the kernel signature (``extern "C" __global__``, parameters in
runtime-parameter order, ``:449-462``), the float literal spelling (``:67-83``)
and the per-element arithmetic (same C expressions, so elementwise results are
bit-identical to the reference's kernels: ``:306-392``).

What differs is the execution model.  The reference runs one thread per logical
block element (``:122-126``, ``block_shapes.py:104-114``).  Here a CTA of ``T``
threads owns the whole logical block and every thread holds ``E`` elements of
each block value in registers:

* layout: element ``L`` of a (row-major flattened) shape lives in thread
  ``(L / V) % T``, register ``(L / (V*T)) * V + L % V`` — ``V`` consecutive
  elements per thread so a contiguous access becomes one 128-bit ld/st;
* every block value is emitted per *context* (the shape it is consumed in, plus
  which context axis each of its axes maps to), so ``[BM,1]`` and ``[1,BN]``
  index vectors are simply re-evaluated in the ``[BM,BN]`` context that uses
  them, and kernels may mix unrelated tile shapes (``tl.dot`` operands);
* loads/stores: contiguity along the fast axis is proven statically from an
  affine analysis of the offset expression; alignment and "whole vector
  in-bounds" are tested per 16-byte group at run time, falling back to
  predicated scalar accesses for the ragged edge;
* reductions: per-thread partial -> ``__shfl_xor_sync`` butterfly -> one shared
  slot per warp -> every thread combines the slots in a fixed order
  (deterministic, one barrier) instead of the reference's shared-memory tree
  with ``log2(width)+1`` barriers (``:183-232``);
* softmax's max -> exp -> sum chain may be fused into one online (max, sum)
  reduction (``online_softmax=True``);
* a runtime loop whose body is ``acc = tl.dot(load A-tile, load B-tile, acc)``
  is handed to the TMA/tcgen05 GEMM generator (dot_codegen.py); any other
  ``tl.dot`` takes a shared-memory SIMT path.
"""

from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass, field
from typing import Any

from .block_shapes import broadcast_shapes, cuda_kernel_block_shape, prod
from .nodes import Const, Param
from .ssa import SSAForRange, SSAItem, SSAOp, SSAOperand, SSAValue
from .types import (
    BF16, BOOL, BYTE_WIDTH, F8E4M3, F8E5M2, F16, F32, FLOAT_UNARY, HALF_WIDTH, I32, BlockType, PointerType, ScalarType, Type, element_of, shape_of,
)

# --------------------------------------------------------------------------- artefacts


@dataclass
class LaunchPlan:
    """Everything the runtime needs besides the source text."""

    kernel_name: str
    threads: int
    dynamic_smem: int = 0
    kind: str = "simt"          # "simt": launched on the caller's grid as is;
                                # "tcgen05": persistent GEMM — dot_codegen.prepare_launch builds
                                # the tensor maps, the CUDA grid and the trailing arguments
    cluster: tuple[int, int, int] = (1, 1, 1)
    notes: dict[str, Any] = field(default_factory=dict)


@dataclass
class KernelArtifact:
    src: str
    plan: LaunchPlan


# --------------------------------------------------------------------------- contexts


@dataclass(frozen=True)
class Ctx:
    """A consumption context: full shape plus, for the value at hand, the context
    axis each of its own axes corresponds to."""

    shape: tuple[int, ...]
    amap: tuple[int, ...]


def _operand_ctx(ctx: Ctx, result_rank: int, operand_rank: int) -> Ctx:
    """Context of a right-aligned (NumPy broadcast) operand of an op emitted in ``ctx``."""
    shift = result_rank - operand_rank
    return Ctx(ctx.shape, tuple(ctx.amap[shift + a] for a in range(operand_rank)))


@dataclass
class _Layout:
    """Register layout of one full shape over the CTA's threads."""

    index: int
    shape: tuple[int, ...]
    threads: int
    vec: int
    regs: int
    guarded: bool  # some (thread, register) slots fall outside the shape

    @property
    def numel(self) -> int:
        return prod(self.shape)


@dataclass
class _Inst:
    """One emitted instance of an SSA value."""

    kind: str                  # "scalar" | "array" | "ptr"
    text: str = ""             # scalar: C expression / variable; array: array name
    base: str = ""             # ptr: parameter name
    index: "_Inst | None" = None   # ptr: index instance (scalar or array), None = 0
    elem: ScalarType | None = None  # ptr: pointee type

    def at(self, r: str) -> str:
        return self.text if self.kind == "scalar" else f"{self.text}[{r}]"


_BOUNDS_HELPERS = '''\
static __device__ __forceinline__ __attribute__((unused)) void mtb_oob_report(
        unsigned* status, unsigned parameter, long long index) {
    // the first offender wins: word 0 = 0xB0000000 | parameter position, words 1-2 = the index
    if (atomicCAS(status, 0u, 0xB0000000u | parameter) == 0u) {
        status[1] = (unsigned)((unsigned long long)index & 0xffffffffull);
        status[2] = (unsigned)((unsigned long long)index >> 32);
    }
}
template <typename T>
static __device__ __forceinline__ __attribute__((unused)) T mtb_ck_ld(
        const T* base, long long index, long long extent, unsigned* status, unsigned parameter) {
    if (index >= 0 && index < extent) return *reinterpret_cast<const volatile T*>(base + index);
    mtb_oob_report(status, parameter, index);
    return T(0);
}
template <typename T, typename V>
static __device__ __forceinline__ __attribute__((unused)) void mtb_ck_st(
        T* base, long long index, long long extent, unsigned* status, unsigned parameter, V value) {
    if (index >= 0 && index < extent) base[index] = (T)value;
    else mtb_oob_report(status, parameter, index);
}
template <typename T, typename V>
static __device__ __forceinline__ __attribute__((unused)) void mtb_ck_atomic_add(
        T* base, long long index, long long extent, unsigned* status, unsigned parameter, V value) {
    if (index >= 0 && index < extent) atomicAdd(base + index, (T)value);
    else mtb_oob_report(status, parameter, index);
}
'''

_HALF_HELPERS = '''\
static __device__ __forceinline__ __attribute__((unused)) unsigned short mtb_f32_to_bf16(float f) {
    unsigned short h;
    asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(f));
    return h;
}
static __device__ __forceinline__ __attribute__((unused)) unsigned short mtb_f32_to_f16(float f) {
    unsigned short h;
    asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f));
    return h;
}
static __device__ __forceinline__ __attribute__((unused)) float mtb_f16_to_f32(unsigned short h) {
    float f;
    asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h));
    return f;
}
static __device__ __forceinline__ __attribute__((unused)) float mtb_round_f16(float f) {
    return mtb_f16_to_f32(mtb_f32_to_f16(f));
}
static __device__ __forceinline__ __attribute__((unused)) float mtb_round_bf16(float f) {
    return __uint_as_float(((unsigned)mtb_f32_to_bf16(f)) << 16);
}
static __device__ __forceinline__ __attribute__((unused)) float mtb_e4m3_to_f32(unsigned char v) {
    unsigned pair;                       // the low byte converts into the low half
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"((unsigned short)v));
    return mtb_f16_to_f32((unsigned short)(pair & 0xffffu));
}
static __device__ __forceinline__ __attribute__((unused)) unsigned char mtb_f32_to_e4m3(float f) {
    unsigned short pair;                 // second source -> low byte; saturates to +-448, keeps NaN
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(0.0f), "f"(f));
    return (unsigned char)(pair & 0xffu);
}
static __device__ __forceinline__ __attribute__((unused)) float mtb_e5m2_to_f32(unsigned char v) {
    unsigned pair;
    asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(pair) : "h"((unsigned short)v));
    return mtb_f16_to_f32((unsigned short)(pair & 0xffffu));
}
static __device__ __forceinline__ __attribute__((unused)) unsigned char mtb_f32_to_e5m2(float f) {
    unsigned short pair;
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(0.0f), "f"(f));
    return (unsigned char)(pair & 0xffu);
}'''

_IDENTITY = {
    ("sum", F32): "0.0f", ("sum", I32): "0",
    ("max", F32): "(-__int_as_float(0x7f800000))", ("max", I32): "(-2147483647 - 1)",
    ("min", F32): "__int_as_float(0x7f800000)", ("min", I32): "2147483647",
}


class SSACUDACodegen:
    BINARY_OPS = {"add": "+", "sub": "-", "mul": "*", "div": "/", "rem": "%", "cmp_lt": "<", "and": "&&"}
    ELEMENTWISE = {
        "add", "sub", "mul", "div", "rem", "cmp_lt", "and", "maximum", "minimum", "neg", "not", "exp",
        "select", "load", "addptr", "full", "zeros", "empty", "arange", *FLOAT_UNARY,
    }

    def __init__(
        self,
        num_warps: int | None = None,
        elems_per_thread: int = 8,
        max_vec: int = 4,
        online_softmax: bool = False,
        streaming: bool = True,
        num_stages: int | None = None,
        cta_group: int | None = None,
        min_ctas_per_sm: int | None = None,
        group_m: int | None = None,
        tensor_cores: bool = True,
        a_rows: int | None = None,
        cta_rows: int | None = None,
        tile_n: int | None = None,
        split_k: int | None = None,
        bounds_check: bool = False,
    ) -> None:
        self.num_warps = num_warps
        self.elems_per_thread = elems_per_thread
        self.max_vec = max_vec
        self.online_softmax = online_softmax
        self.streaming = streaming
        self.num_stages = num_stages
        self.cta_group = cta_group
        self.min_ctas_per_sm = min_ctas_per_sm
        self.group_m = group_m
        self.tensor_cores = tensor_cores      # False: tl.dot loops stay on the SIMT path
        self.a_rows = a_rows                  # tl.dot: rows of A the skinny variant fetches
        self.cta_rows = cta_rows              # tl.dot: rows of C per CTA of a pair (128 or 256)
        self.tile_n = tile_n                  # tl.dot: columns of the kernel's own tile (64, 128 or 256)
        self.split_k = split_k                # tl.dot: units of work per tile along K (single-CTA kernel)
        # Debug mode: every global access is compared with the array's extent, which the
        # launcher passes beside the pointers.  An access outside it is skipped (a load gives
        # zero) and the first one is recorded in a status word; nothing traps.  Accesses are
        # made element by element and tl.dot loops stay on the SIMT path so that each of them
        # goes through the check.
        self.bounds_check = bounds_check
        if bounds_check:
            self.max_vec = 1
            self.online_softmax = False
            self.tensor_cores = False
        self._reset()

    def _reset(self) -> None:
        self.lines: list[str] = []
        self.shared_lines: list[str] = []
        self.indent = 1
        self.defs: dict[int, SSAOp] = {}
        self.types: dict[int, Type] = {}
        self.affine: dict[int, tuple[int | None, ...]] = {}
        self.demand: dict[int, list[Ctx]] = {}
        self.inst: dict[tuple[int, Ctx | None], _Inst] = {}
        self.foreign: dict[int, list[Ctx]] = {}     # register-held values also needed in other shapes
        self.layouts: dict[tuple[int, ...], _Layout] = {}
        self.threads = 1
        self.loop_depth = 0
        self.uses_half_helpers = False
        self.dynamic_smem = 0
        self._open: tuple[_Layout, list[str], list[str]] | None = None
        self._tmp = 0

    # ------------------------------------------------------------------ small helpers

    def cuda_type(self, ty: Type) -> str:
        element = element_of(ty)
        if element == I32:
            return "int"
        if element in (F32, BF16, F16) + BYTE_WIDTH:
            return "float"       # narrow storage types are widened to fp32 in registers
        if element == BOOL:
            return "bool"
        if isinstance(element, PointerType):
            if element.element in BYTE_WIDTH:
                return "unsigned char*"
            return "unsigned short*" if element.element in HALF_WIDTH else f"{self.cuda_type(element.element)}*"
        raise TypeError(f"Cannot lower CUDA type: {ty}")

    def literal(self, value: object) -> str:
        if isinstance(value, bool):
            return "true" if value else "false"
        if isinstance(value, float):
            if math.isnan(value):
                return "__int_as_float(0x7fc00000)"
            if math.isinf(value):
                positive = "__int_as_float(0x7f800000)"
                return positive if value > 0 else f"(-{positive})"
            return f"{value}f"
        if isinstance(value, int):
            return str(value)
        raise TypeError(f"Unsupported CUDA literal: {value!r}")

    def _line(self, text: str) -> None:
        self.lines.append("    " * self.indent + text)

    def _fresh(self, stem: str) -> str:
        self._tmp += 1
        return f"{stem}{self._tmp}"

    def _type_of(self, operand: SSAOperand) -> Type | None:
        if operand is None:
            return None
        if isinstance(operand, (SSAValue, Param)):
            return operand.ty
        if isinstance(operand.value, bool):
            return BOOL
        return I32 if isinstance(operand.value, int) else F32

    # ------------------------------------------------------------------ analysis passes

    def _index_ops(self, ops: list[SSAItem]) -> None:
        for op in ops:
            if isinstance(op, SSAForRange):
                for value in (op.index, *op.carried_args, *op.results):
                    self.types[value.id] = value.ty
                self._index_ops(op.body)
            elif op.result is not None:
                self.defs[op.result.id] = op
                self.types[op.result.id] = op.result.ty

    def _affine_of(self, operand: SSAOperand, rank: int) -> tuple[int | None, ...]:
        """Per-axis d(value)/d(coordinate), right-aligned to ``rank`` axes."""
        own: tuple[int | None, ...] = ()
        if isinstance(operand, SSAValue):
            own = self.affine.get(operand.id, tuple([None] * len(shape_of(operand.ty))))
        return (0,) * (rank - len(own)) + own

    def _analyse_affine(self, ops: list[SSAItem]) -> None:
        for op in ops:
            if isinstance(op, SSAForRange):
                self.affine[op.index.id] = ()
                # A carried block keeps its per-axis coefficients when every iteration only adds
                # something uniform to it (`cols += BLOCK`, `ptrs += BK * stride`): assume the
                # initial value's coefficients, analyse the body, and keep the assumption only
                # for the slots whose yield confirms it.
                assumed = {}
                for initial, arg in zip(op.carried_inputs, op.carried_args):
                    rank = len(shape_of(arg.ty))
                    assumed[arg.id] = self._affine_of(initial, rank) if isinstance(initial, SSAValue) \
                        else (0,) * rank
                for attempt in range(2):
                    for arg in op.carried_args:
                        self.affine[arg.id] = assumed[arg.id]
                    self._analyse_affine(op.body)
                    stable = True
                    for arg, yielded in zip(op.carried_args, op.yields):
                        rank = len(shape_of(arg.ty))
                        after = self._affine_of(yielded, rank) if isinstance(yielded, SSAValue) else (0,) * rank
                        if after != assumed[arg.id]:
                            assumed[arg.id] = tuple(0 if d == 1 else None for d in shape_of(arg.ty))
                            stable = False
                    if stable:
                        break
                for arg, result in zip(op.carried_args, op.results):
                    self.affine[result.id] = assumed[arg.id]
                continue
            if op.result is None:
                continue
            shape = shape_of(op.result.ty)
            rank = len(shape)
            code = op.opcode
            unknown = tuple(0 if d == 1 else None for d in shape)
            if code == "arange":
                coefs: tuple[int | None, ...] = (1,)
            elif code == "expand_dims":
                inner = list(self._affine_of(op.operands[0], rank - 1))
                inner.insert(op.attrs["axis"], 0)
                coefs = tuple(inner)
            elif code == "trans":
                inner = self._affine_of(op.operands[0], 2)
                coefs = (inner[1], inner[0])
            elif code in ("add", "sub", "addptr"):
                a = self._affine_of(op.operands[0], rank)
                b = self._affine_of(op.operands[1], rank)
                sign = -1 if code == "sub" else 1
                coefs = tuple(
                    None if x is None or y is None else x + sign * y for x, y in zip(a, b)
                )
            elif code == "mul":
                a = self._affine_of(op.operands[0], rank)
                b = self._affine_of(op.operands[1], rank)
                ca, cb = (self._int_const(x) for x in op.operands[:2])
                if cb is not None:
                    coefs = tuple(None if x is None else x * cb for x in a)
                elif ca is not None:
                    coefs = tuple(None if y is None else y * ca for y in b)
                else:
                    coefs = tuple(0 if x == 0 and y == 0 else None for x, y in zip(a, b))
            elif code in ("full", "zeros", "program_id", "num_programs"):
                coefs = (0,) * rank
            else:
                coefs = unknown
            self.affine[op.result.id] = tuple(
                0 if d == 1 else c for c, d in zip(coefs, shape)
            ) if rank else ()

    @staticmethod
    def _int_const(operand: SSAOperand) -> int | None:
        if isinstance(operand, Const) and type(operand.value) is int:
            return operand.value
        return None

    def _want(self, operand: SSAOperand, ctx: Ctx | None) -> None:
        if not isinstance(operand, SSAValue) or not isinstance(operand.ty, BlockType):
            return
        assert ctx is not None
        wanted = self.demand.setdefault(operand.id, [])
        if ctx not in wanted:
            wanted.append(ctx)

    @staticmethod
    def _own_ctx(ty: Type) -> Ctx:
        shape = shape_of(ty)
        return Ctx(shape, tuple(range(len(shape))))

    def _analyse_demand(self, ops: list[SSAItem]) -> None:
        """Backward walk: which contexts must each block value be available in?"""
        for op in reversed(ops):
            if isinstance(op, SSAForRange):
                for result in op.results:
                    self._check_materialised(result)
                for yielded, result in zip(op.yields, op.results):
                    self._want(yielded, self._own_ctx(result.ty))
                self._analyse_demand(op.body)
                for arg in op.carried_args:
                    self._check_materialised(arg)
                for initial, result in zip(op.carried_inputs, op.results):
                    self._want(initial, self._own_ctx(result.ty))
                continue
            code = op.opcode
            if code == "break_unless":
                continue                      # reads one scalar
            if code in ("store", "atomic_add"):
                shapes = [shape_of(self._type_of(x)) for x in op.operands if x is not None]
                full = broadcast_shapes(*shapes) if any(shapes) else ()
                if full:
                    ctx = Ctx(full, tuple(range(len(full))))
                    for operand in op.operands:
                        rank = len(shape_of(self._type_of(operand))) if operand is not None else 0
                        self._want(operand, _operand_ctx(ctx, len(full), rank))
                continue
            result = op.result
            assert result is not None
            if code in ("sum", "max", "min"):
                self._want(op.operands[0], self._own_ctx(op.operands[0].ty))
                continue
            if code == "dot":
                self._check_materialised(result)
                for operand in op.operands:
                    if operand is not None:
                        self._want(operand, self._own_ctx(self._type_of(operand)))
                continue
            if not isinstance(result.ty, BlockType):
                continue
            rank = result.ty.rank
            for ctx in self.demand.get(result.id, []):
                if code == "expand_dims":
                    axis = op.attrs["axis"]
                    amap = tuple(ctx.amap[a if a < axis else a + 1] for a in range(rank - 1))
                    self._want(op.operands[0], Ctx(ctx.shape, amap))
                elif code == "trans":
                    # the operand's axes stand where the result's stand, exchanged
                    self._want(op.operands[0], Ctx(ctx.shape, (ctx.amap[1], ctx.amap[0])))
                else:
                    for operand in op.operands:
                        operand_rank = len(shape_of(self._type_of(operand))) if operand is not None else 0
                        self._want(operand, _operand_ctx(ctx, rank, operand_rank))

    def _check_materialised(self, value: SSAValue) -> None:
        """Loop-carried values and dot results live in registers in their own layout."""
        if not isinstance(value.ty, BlockType):
            return
        own = self._own_ctx(value.ty)
        foreign = [ctx for ctx in self.demand.get(value.id, []) if ctx != own]
        if foreign:
            # used in another shape (a carried row vector broadcast over a tile): it is
            # redistributed through shared memory where it is defined
            if isinstance(element_of(value.ty), PointerType):
                raise TypeError(f"{value} : {value.ty} is held in registers and cannot be broadcast")
            if prod(own.shape) * 4 > 48 * 1024:
                raise TypeError(
                    f"{value} : {value.ty} is held in registers and cannot be broadcast "
                    f"into a {'x'.join(map(str, foreign[0].shape))} block"
                )
            self.foreign[value.id] = foreign
        self.demand[value.id] = [own]

    # ------------------------------------------------------------------ layouts

    def _choose_threads(self) -> int:
        sizes = [prod(ctx.shape) for ctxs in self.demand.values() for ctx in ctxs]
        if not sizes:
            return 1
        largest = max(sizes)
        if self.num_warps is not None:
            return max(1, min(1024, self.num_warps * 32))
        if largest < 32:
            return largest
        want = -(-largest // self.elems_per_thread)
        want = 1 << (want - 1).bit_length()          # next power of two
        return max(32, min(1024, want))

    def _layout(self, shape: tuple[int, ...]) -> _Layout:
        layout = self.layouts.get(shape)
        if layout is None:
            numel, threads = prod(shape), self.threads
            vec = self.max_vec
            while vec > 1 and (shape[-1] % vec or numel < threads * vec):
                vec //= 2
            groups = -(-numel // (threads * vec))
            regs = groups * vec
            layout = _Layout(len(self.layouts), shape, threads, vec, regs,
                             guarded=regs * threads != numel)
            self.layouts[shape] = layout
            self._emit_layout_prologue(layout)
        return layout

    def _emit_layout_prologue(self, lay: _Layout) -> None:
        k = lay.index
        self._flush()
        self._line(f"int L{k}[{lay.regs}];")
        self._line("#pragma unroll")
        self._line(
            f"for (int r = 0; r < {lay.regs}; ++r) "
            f"L{k}[r] = ((r / {lay.vec}) * {lay.threads} + (int)threadIdx.x) * {lay.vec} + (r % {lay.vec});"
        )

    def _coord(self, lay: _Layout, axis: int, r: str) -> str:
        linear = f"L{lay.index}[{r}]"
        if len(lay.shape) == 1:
            return linear
        inner = lay.shape[1]
        return f"({linear} / {inner})" if axis == 0 else f"({linear} % {inner})"

    def _valid(self, lay: _Layout, r: str) -> str | None:
        return f"(L{lay.index}[{r}] < {lay.numel})" if lay.guarded else None

    # ------------------------------------------------------------------ fused elementwise loops

    def _stmt(self, lay: _Layout, decl: str | None, body: str) -> None:
        """Queue ``body`` (uses loop variable ``r``) into the open per-register loop."""
        if self._open is not None and self._open[0] is not lay:
            self._flush()
        if self._open is None:
            self._open = (lay, [], [])
        if decl:
            self._open[1].append(decl)
        self._open[2].append(body)

    def _flush(self) -> None:
        if self._open is None:
            return
        lay, decls, body = self._open
        self._open = None
        for decl in decls:
            self._line(decl)
        self._line("#pragma unroll")
        self._line(f"for (int r = 0; r < {lay.regs}; ++r) {{")
        self.indent += 1
        for statement in body:
            self._line(statement)
        self.indent -= 1
        self._line("}")

    # ------------------------------------------------------------------ operand access

    def _get(self, operand: SSAOperand, ctx: Ctx | None) -> _Inst:
        if isinstance(operand, Const):
            return _Inst("scalar", self.literal(operand.value))
        if isinstance(operand, Param):
            if isinstance(operand.ty, PointerType):
                return _Inst("ptr", base=operand.name, index=None, elem=operand.ty.element)
            return _Inst("scalar", operand.name)
        assert isinstance(operand, SSAValue)
        key = (operand.id, ctx if isinstance(operand.ty, BlockType) else None)
        found = self.inst.get(key)
        if found is None:
            raise RuntimeError(f"SSA value {operand} is not defined")
        return found

    def _operand_inst(self, op: SSAOp, position: int, ctx: Ctx | None) -> _Inst | None:
        operand = op.operands[position]
        if operand is None:
            return None
        if ctx is None or not isinstance(self._type_of(operand), BlockType):
            return self._get(operand, None)
        result_rank = len(shape_of(op.result.ty)) if op.result is not None else len(ctx.shape)
        operand_rank = len(shape_of(self._type_of(operand)))
        return self._get(operand, _operand_ctx(ctx, result_rank, operand_rank))

    # ------------------------------------------------------------------ expression text

    def _expr(self, op: SSAOp, args: list[str], result_ty: Type) -> str:
        code = op.opcode
        if code in self.BINARY_OPS:
            return f"({args[0]} {self.BINARY_OPS[code]} {args[1]})"
        if code in ("maximum", "minimum"):
            symbol = ">" if code == "maximum" else "<"
            lhs, rhs = args
            if element_of(result_ty) == F32:
                # an integer operand of a mixed maximum/minimum is converted first, so that
                # isnan() sees a float (isnan(int) is ambiguous) and both arms have one type
                lhs, rhs = (text if element_of(self._type_of(operand)) == F32 else f"(float)({text})"
                            for text, operand in zip((lhs, rhs), op.operands))
            pick = f"(({lhs}) {symbol} ({rhs}) ? ({lhs}) : ({rhs}))"
            if element_of(result_ty) == F32:
                pick = f"(isnan({lhs}) ? ({lhs}) : (isnan({rhs}) ? ({rhs}) : {pick}))"
            return pick
        if code == "neg":
            return f"-({args[0]})"
        if code == "not":
            return f"!({args[0]})"
        if code == "exp":
            if element_of(result_ty) != F32:
                raise TypeError(f"exp requires f32, got {result_ty}")
            return f"expf({args[0]})"
        if code == "select":
            return f"({args[0]} ? {args[1]} : {args[2]})"
        if code == "abs" and element_of(result_ty) == I32:
            return f"(({args[0]}) < 0 ? -({args[0]}) : ({args[0]}))"
        if code in FLOAT_UNARY:
            if element_of(result_ty) != F32:
                raise TypeError(f"{code} requires f32, got {result_ty}")
            if code.startswith("round_"):
                self.uses_half_helpers = True
            return f"{FLOAT_UNARY[code]}({args[0]})"
        raise TypeError(f"Unsupported SSA opcode: {code}")

    # ------------------------------------------------------------------ emission: scalars

    def _emit_scalar(self, op: SSAOp) -> None:
        result = op.result
        assert result is not None
        code = op.opcode
        name = f"v{result.id}"
        if code == "program_id":
            axis = op.attrs["axis"]
            if axis not in (0, 1, 2):
                raise ValueError(f"Invalid program axis: {axis}")
            self._flush()
            self._line(f"int {name} = {self._program_id(axis)};")
        elif code == "num_programs":
            axis = op.attrs["axis"]
            if axis not in (0, 1, 2):
                raise ValueError(f"Invalid program axis: {axis}")
            self._flush()
            self._line(f"int {name} = (int)gridDim.{'xyz'[axis]};")
        elif code == "addptr":
            base = self._get(op.operands[0], None)
            offset = self._get(op.operands[1], None)
            index = offset if base.index is None else _Inst(
                "scalar", f"({base.index.text} + {offset.text})"
            )
            self.inst[(result.id, None)] = _Inst("ptr", base=base.base, index=index, elem=base.elem)
            return
        elif code == "load":
            self._flush()
            ptr = self._get(op.operands[0], None)
            mask = self._operand_inst(op, 1, None)
            other = self._operand_inst(op, 2, None)
            fallback = other.text if other else ("0.0f" if element_of(result.ty) != I32 else "0")
            where = ptr.index.text if ptr.index is not None else "0"
            condition = mask.text if mask else "true"
            # A scalar is one value for the whole program, and loop bounds, `while` conditions
            # and the barriers inside reductions rely on every thread of the CTA holding the
            # same one.  So one thread reads it (a volatile read: the word may be a flag
            # that another program updates with tl.atomic_add, or this program's own earlier
            # scalar store, which that same thread made) and hands it to the others through
            # shared memory.  The leading barrier orders the read after block stores made by
            # other threads of the CTA and keeps the slot from being rewritten while a slower
            # thread still reads the previous value.
            storage = ("unsigned char" if ptr.elem in BYTE_WIDTH else
                       "unsigned short" if ptr.elem in HALF_WIDTH else self.cuda_type(ptr.elem))
            source = ptr if self.bounds_check else dataclasses.replace(
                ptr, base=f"((volatile {storage}*){ptr.base})")      # the checked read is volatile already
            read = self._read(source, where)
            cty = self.cuda_type(result.ty)
            slot = f"uni_{result.id}"
            self.shared_lines.append(f"    __shared__ {cty} {slot};")
            self._line("__syncthreads();")
            self._line(f"if (threadIdx.x == 0) {{ {slot} = ({condition} ? {read} : {fallback}); }}")
            self._line("__syncthreads();")
            self._line(f"{cty} {name} = {slot};")
        else:
            args = [self._get(x, None).text for x in op.operands if x is not None]
            self._flush()
            self._line(f"{self.cuda_type(result.ty)} {name} = {self._expr(op, args, result.ty)};")
        self.inst[(result.id, None)] = _Inst("scalar", name)

    def _program_id(self, axis: int) -> str:
        return "(int)blockIdx." + "xyz"[axis]

    def _checked(self, helper: str, ptr: _Inst, where: str, value: str | None = None) -> str:
        """The bounds-checked form of one access to ``ptr.base[where]``."""
        position = self.param_positions[ptr.base]
        tail = "" if value is None else f", {value}"
        return (f"{helper}({ptr.base}, (long long)({where}), mtb_ext_{ptr.base}, mtb_oob, "
                f"{position}u{tail})")

    def _read(self, ptr: _Inst, where: str) -> str:
        raw = self._checked("mtb_ck_ld", ptr, where) if self.bounds_check else f"{ptr.base}[{where}]"
        if ptr.elem == BF16:
            return f"__uint_as_float(((unsigned)({raw})) << 16)"
        if ptr.elem == F16:
            self.uses_half_helpers = True
            return f"mtb_f16_to_f32({raw})"
        if ptr.elem in BYTE_WIDTH:
            self.uses_half_helpers = True
            return f"mtb_{'e4m3' if ptr.elem == F8E4M3 else 'e5m2'}_to_f32({raw})"
        return raw

    # ------------------------------------------------------------------ emission: block values

    def _emit_block(self, op: SSAOp, ctx: Ctx) -> None:
        result = op.result
        assert result is not None and isinstance(result.ty, BlockType)
        lay = self._layout(ctx.shape)
        code = op.opcode
        cty = self.cuda_type(result.ty)
        name = f"v{result.id}_{lay.index}" + ("" if ctx.amap == tuple(range(len(ctx.shape))) else
                                              "_" + "".join(map(str, ctx.amap)))
        key = (result.id, ctx)

        if code == "expand_dims":
            axis = op.attrs["axis"]
            rank = result.ty.rank
            amap = tuple(ctx.amap[a if a < axis else a + 1] for a in range(rank - 1))
            self.inst[key] = self._get(op.operands[0], Ctx(ctx.shape, amap))
            return
        if code == "trans":
            self.inst[key] = self._get(op.operands[0], Ctx(ctx.shape, (ctx.amap[1], ctx.amap[0])))
            return
        if code == "addptr":
            base = self._operand_inst(op, 0, ctx)
            offset = self._operand_inst(op, 1, ctx)
            assert base is not None and offset is not None
            if base.index is None:
                index = offset
            else:
                self._stmt(lay, f"int {name}[{lay.regs}];",
                           f"{name}[r] = {base.index.at('r')} + {offset.at('r')};")
                index = _Inst("array", name)
            self.inst[key] = _Inst("ptr", base=base.base, index=index, elem=base.elem)
            return
        if code == "arange":
            (axis,) = ctx.amap
            start = op.attrs["start"]
            coord = self._coord(lay, axis, "r")
            value = coord if start == 0 else f"({start} + {coord})"
            self._stmt(lay, f"int {name}[{lay.regs}];", f"{name}[r] = {value};")
        elif code in ("zeros", "empty"):
            zero = self.literal(False if cty == "bool" else 0.0 if cty == "float" else 0)
            self._stmt(lay, f"{cty} {name}[{lay.regs}];", f"{name}[r] = {zero};")
        elif code == "full":
            fill = self._get(op.operands[0], None).text
            self._stmt(lay, f"{cty} {name}[{lay.regs}];", f"{name}[r] = {fill};")
        elif code == "load":
            self._emit_load(op, ctx, lay, name)
        else:
            args = []
            for position, operand in enumerate(op.operands):
                inst = self._operand_inst(op, position, ctx)
                assert inst is not None
                args.append(inst.at("r"))
            self._stmt(lay, f"{cty} {name}[{lay.regs}];",
                       f"{name}[r] = {self._expr(op, args, result.ty)};")
        self.inst[key] = _Inst("array", name)

    def _fast_axis_coef(self, operand: SSAOperand, ctx: Ctx) -> int | None:
        """d(index)/d(fast context coordinate) of a pointer operand seen in ``ctx``."""
        ty = self._type_of(operand)
        shape = shape_of(ty)
        if not shape:
            return 0
        fast = len(ctx.shape) - 1
        coefs = self._affine_of(operand, len(shape))
        for axis, target in enumerate(ctx.amap):
            if target == fast:
                return 0 if shape[axis] == 1 else coefs[axis]
        return 0

    def _emit_load(self, op: SSAOp, ctx: Ctx, lay: _Layout, name: str) -> None:
        result = op.result
        assert result is not None
        ptr = self._operand_inst(op, 0, ctx)
        mask = self._operand_inst(op, 1, ctx)
        other = self._operand_inst(op, 2, ctx)
        assert ptr is not None
        cty = self.cuda_type(result.ty)
        zero = "0" if cty == "int" else "0.0f"

        def fallback(r: str) -> str:
            return other.at(r) if other is not None else zero

        def predicate(r: str) -> str:
            terms = [t for t in (mask.at(r) if mask else None, self._valid(lay, r)) if t]
            return " && ".join(terms) if terms else "true"

        def where(r: str) -> str:
            return ptr.index.at(r) if ptr.index is not None else "0"

        ptr_rank = len(shape_of(self._type_of(op.operands[0])))
        ptr_ctx = _operand_ctx(ctx, result.ty.rank, ptr_rank)
        vector = (
            lay.vec > 1
            and ptr.elem == F32
            and self._fast_axis_coef(op.operands[0], ptr_ctx) == 1
        )
        if not vector:
            self._stmt(lay, f"{cty} {name}[{lay.regs}];",
                       f"{name}[r] = ({predicate('r')} ? {self._read(ptr, where('r'))} : {fallback('r')});")
            return

        self._flush()
        v = lay.vec
        vec_t = {4: "float4", 2: "float2"}[v]
        fields = "xyzw"[:v]
        self._line(f"{cty} {name}[{lay.regs}];")
        self._line("#pragma unroll")
        self._line(f"for (int g = 0; g < {lay.regs}; g += {v}) {{")
        self.indent += 1
        self._line(f"const float* p = {ptr.base} + {where('g')};")
        whole = " && ".join(f"({predicate(f'g + {e}')})" for e in range(v))
        self._line(f"if (({whole}) && ((reinterpret_cast<unsigned long long>(p) & {4 * v - 1}ull) == 0ull)) {{")
        self.indent += 1
        if self.streaming:
            self._line(f"const {vec_t} q = __ldcs(reinterpret_cast<const {vec_t}*>(p));")
        else:
            self._line(f"const {vec_t} q = *reinterpret_cast<const {vec_t}*>(p);")
        for e in range(v):
            self._line(f"{name}[g + {e}] = q.{fields[e]};")
        self.indent -= 1
        self._line("} else {")
        self.indent += 1
        self._line("#pragma unroll")
        self._line(f"for (int e = 0; e < {v}; ++e) {{")
        self.indent += 1
        self._line("const int r = g + e;")
        self._line(f"{name}[r] = ({predicate('r')} ? {self._read(ptr, where('r'))} : {fallback('r')});")
        self.indent -= 1
        self._line("}")
        self.indent -= 1
        self._line("}")
        self.indent -= 1
        self._line("}")

    # ------------------------------------------------------------------ emission: stores

    def _convert_for_store(self, text: str, value_ty: Type | None, elem: ScalarType) -> str:
        have = element_of(value_ty) if value_ty is not None else None
        if elem == BF16:
            self.uses_half_helpers = True
            return f"mtb_f32_to_bf16((float)({text}))"
        if elem == F16:
            self.uses_half_helpers = True
            return f"mtb_f32_to_f16((float)({text}))"
        if elem in BYTE_WIDTH:
            self.uses_half_helpers = True
            return f"mtb_f32_to_{'e4m3' if elem == F8E4M3 else 'e5m2'}((float)({text}))"
        if elem == F32 and have == I32:
            return f"(float)({text})"
        if elem == I32 and have in (F32, BF16, F16) + BYTE_WIDTH:
            return f"(int)({text})"
        return text

    def _emit_store(self, op: SSAOp) -> None:
        shapes = [shape_of(self._type_of(x)) for x in op.operands if x is not None]
        full = broadcast_shapes(*shapes) if any(shapes) else ()
        value_ty = self._type_of(op.operands[1])
        atomic = op.opcode == "atomic_add"

        def write(pointer: _Inst, index: str, converted: str) -> str:
            if self.bounds_check:
                return self._checked("mtb_ck_atomic_add" if atomic else "mtb_ck_st", pointer, index, converted) + ";"
            target = f"{pointer.base}[{index}]"
            return f"atomicAdd(&{target}, {converted});" if atomic else f"{target} = {converted};"

        if not full:
            self._flush()
            ptr = self._get(op.operands[0], None)
            value = self._get(op.operands[1], None).text
            mask = self._get(op.operands[2], None).text if op.operands[2] is not None else None
            where = ptr.index.text if ptr.index is not None else "0"
            text = write(ptr, where, self._convert_for_store(value, value_ty, ptr.elem))
            guard = "threadIdx.x == 0" + (f" && {mask}" if mask else "")
            self._line(f"if ({guard}) {{ {text} }}")
            # one thread wrote on behalf of the program: loads that other threads make later
            # must not overtake it
            self._line("__syncthreads();")
            return

        ctx = Ctx(full, tuple(range(len(full))))
        lay = self._layout(full)

        def inst_of(position: int) -> _Inst | None:
            operand = op.operands[position]
            if operand is None:
                return None
            rank = len(shape_of(self._type_of(operand)))
            if rank == 0:
                return self._get(operand, None)
            return self._get(operand, _operand_ctx(ctx, len(full), rank))

        ptr, value, mask = inst_of(0), inst_of(1), inst_of(2)
        assert ptr is not None and value is not None

        def predicate(r: str) -> str:
            terms = [t for t in (mask.at(r) if mask else None, self._valid(lay, r)) if t]
            return " && ".join(terms) if terms else "true"

        def where(r: str) -> str:
            return ptr.index.at(r) if ptr.index is not None else "0"

        def stored(r: str) -> str:
            return self._convert_for_store(value.at(r), value_ty, ptr.elem)

        ptr_rank = len(shape_of(self._type_of(op.operands[0])))
        vector = (
            lay.vec > 1
            and ptr.elem == F32
            and not atomic
            and self._fast_axis_coef(op.operands[0], _operand_ctx(ctx, len(full), ptr_rank)) == 1
        )
        if not vector:
            self._stmt(lay, None, f"if ({predicate('r')}) {{ {write(ptr, where('r'), stored('r'))} }}")
            return

        self._flush()
        v = lay.vec
        vec_t = {4: "float4", 2: "float2"}[v]
        self._line("#pragma unroll")
        self._line(f"for (int g = 0; g < {lay.regs}; g += {v}) {{")
        self.indent += 1
        self._line(f"float* p = {ptr.base} + {where('g')};")
        whole = " && ".join(f"({predicate(f'g + {e}')})" for e in range(v))
        self._line(f"if (({whole}) && ((reinterpret_cast<unsigned long long>(p) & {4 * v - 1}ull) == 0ull)) {{")
        self.indent += 1
        packed = ", ".join(stored(f"g + {e}") for e in range(v))
        if self.streaming:
            self._line(f"__stcs(reinterpret_cast<{vec_t}*>(p), make_{vec_t}({packed}));")
        else:
            self._line(f"*reinterpret_cast<{vec_t}*>(p) = make_{vec_t}({packed});")
        self.indent -= 1
        self._line("} else {")
        self.indent += 1
        self._line("#pragma unroll")
        self._line(f"for (int e = 0; e < {v}; ++e) {{")
        self.indent += 1
        self._line("const int r = g + e;")
        self._line(f"if ({predicate('r')}) {{ {ptr.base}[{where('r')}] = {stored('r')}; }}")
        self.indent -= 1
        self._line("}")
        self.indent -= 1
        self._line("}")
        self.indent -= 1
        self._line("}")

    # ------------------------------------------------------------------ emission: redistribution

    def _emit_redistribution(self, value: SSAValue) -> None:
        """Make a register-held block (loop-carried value, dot result) available in the other
        contexts that consume it: its own layout writes one shared slot per element, every
        consumer layout reads the slots its registers stand for."""
        contexts = self.foreign.get(value.id)
        if not contexts:
            return
        own = self._own_ctx(value.ty)
        lay = self._layout(own.shape)
        source = self.inst[(value.id, own)]
        cty = self.cuda_type(value.ty)
        slots = f"cvt_{value.id}"
        declaration = f"    __shared__ {cty} {slots}[{lay.numel}];"
        if declaration not in self.shared_lines:
            self.shared_lines.append(declaration)
        valid = self._valid(lay, "r")
        write = f"{slots}[L{lay.index}[r]] = {source.at('r')};"
        self._stmt(lay, None, f"if {valid} {{ {write} }}" if valid else write)
        self._flush()
        self._line("__syncthreads();")
        strides = [prod(own.shape[axis + 1:]) for axis in range(len(own.shape))]
        for ctx in contexts:
            target = self._layout(ctx.shape)
            name = f"v{value.id}_{target.index}_" + "".join(map(str, ctx.amap)) + f"_{self._fresh('c')}"
            index = " + ".join(
                f"{self._coord(target, ctx.amap[axis], 'r')} * {strides[axis]}" for axis in range(len(own.shape)))
            guard = self._valid(target, "r")
            read = f"{slots}[{index}]"
            self._stmt(target, f"{cty} {name}[{target.regs}];",
                       f"{name}[r] = {f'({guard} ? {read} : {slots}[0])' if guard else read};")
            self.inst[(value.id, ctx)] = _Inst("array", name)
        self._flush()
        self._line("__syncthreads();")          # the slots may be rewritten (next iteration, next value)

    # ------------------------------------------------------------------ emission: reductions

    def _combine(self, opcode: str, element: ScalarType, lhs: str, rhs: str) -> str:
        if opcode == "sum":
            return f"({lhs} + {rhs})"
        if element == F32:
            return f"{'fmaxf' if opcode == 'max' else 'fminf'}({lhs}, {rhs})"
        symbol = ">" if opcode == "max" else "<"
        return f"({lhs} {symbol} {rhs} ? {lhs} : {rhs})"

    def _emit_reduction(self, op: SSAOp) -> None:
        operand = op.operands[0]
        result = op.result
        assert isinstance(operand, SSAValue) and result is not None
        input_ty = operand.ty
        if not isinstance(input_ty, BlockType) or input_ty.rank != 1:
            raise TypeError(f"{op.opcode} expects a vector input, got {input_ty}")
        if input_ty.size & (input_ty.size - 1):
            raise TypeError(f"reduction width must be a power of two, got {input_ty.size}")
        element = input_ty.element
        if (op.opcode, element) not in _IDENTITY:
            raise TypeError(f"Unsupported type for {op.opcode}: {element}")
        ctx = self._own_ctx(input_ty)
        lay = self._layout(ctx.shape)
        source = self._get(operand, ctx)
        self._flush()
        cty = self.cuda_type(element)
        identity = _IDENTITY[(op.opcode, element)]
        name = f"v{result.id}"
        part = f"part{result.id}"

        def lane_value(r: int) -> str:
            valid = self._valid(lay, str(r))
            return f"({valid} ? {source.at(str(r))} : {identity})" if valid else source.at(str(r))

        self._line(f"{cty} {part} = {lane_value(0)};")
        if lay.regs > 1:
            self._line("#pragma unroll")
            self._line(f"for (int r = 1; r < {lay.regs}; ++r) {{")
            self.indent += 1
            valid = self._valid(lay, "r")
            term = f"({valid} ? {source.at('r')} : {identity})" if valid else source.at("r")
            self._line(f"{part} = {self._combine(op.opcode, element, part, term)};")
            self.indent -= 1
            self._line("}")
        self._emit_cta_combine(op.opcode, element, cty, part, name, str(result.id))
        self.inst[(result.id, None)] = _Inst("scalar", name)

    def _emit_axis_reduction(self, op: SSAOp) -> None:
        """``tl.sum/max/min(x, axis=1)`` of a rank-2 block: one value per row.

        In the block's own layout a row's columns sit in ``cols / vec`` consecutive vector
        slots, i.e. in that many consecutive threads.  When that count is a power of two that
        divides the warp, each thread reduces its vector and a shuffle butterfly over the
        sub-group of lanes leaves the row's result in every slot of the row — which is exactly
        the result broadcast back over the tile (``x - tl.max(x, axis=1)[:, None]``), so that
        use costs nothing more.  Any other use, and any other geometry, goes through one
        shared-memory slot per vector (geometry) or per row (use)."""
        operand, result = op.operands[0], op.result
        assert isinstance(operand, SSAValue) and result is not None
        input_ty = operand.ty
        if op.attrs.get("axis") == 0:
            self._emit_column_reduction(op)
            return
        rows, cols = input_ty.shape
        element = input_ty.element
        if (op.opcode, element) not in _IDENTITY:
            raise TypeError(f"Unsupported type for {op.opcode}: {element}")
        identity, cty = _IDENTITY[(op.opcode, element)], self.cuda_type(element)
        own = self._own_ctx(input_ty)
        lay = self._layout(own.shape)
        source = self._get(operand, own)
        group = cols // lay.vec                   # vector slots (= consecutive threads) per row
        threads = self.threads
        tag = str(result.id)
        self._flush()

        # per-thread: one partial per vector group
        groups = lay.regs // lay.vec
        part = f"rowpart{tag}"
        self._line(f"{cty} {part}[{groups}];")
        self._line("#pragma unroll")
        self._line(f"for (int g = 0; g < {groups}; ++g) {{")
        self.indent += 1
        self._line(f"{cty} acc = {identity};")
        self._line("#pragma unroll")
        self._line(f"for (int e = 0; e < {lay.vec}; ++e) {{")
        self.indent += 1
        self._line(f"const int r = g * {lay.vec} + e;")
        valid = self._valid(lay, "r")
        term = f"({valid} ? {source.at('r')} : {identity})" if valid else source.at("r")
        self._line(f"acc = {self._combine(op.opcode, element, 'acc', term)};")
        self.indent -= 1
        self._line("}")
        self._line(f"{part}[g] = acc;")
        self.indent -= 1
        self._line("}")

        in_warp = (group & (group - 1) == 0 and group <= 32 and threads % group == 0
                   and (threads % 32 == 0 or threads & (threads - 1) == 0))
        broadcast_ctx = Ctx(own.shape, (0,))
        wanted = list(self.demand.get(result.id, []))
        row_totals: _Inst | None = None
        if in_warp:
            if group > 1:
                member_mask = "0xffffffffu" if threads >= 32 else hex((1 << threads) - 1) + "u"
                self._line("#pragma unroll")
                self._line(f"for (int g = 0; g < {groups}; ++g) {{")
                self.indent += 1
                self._line("#pragma unroll")
                self._line(f"for (int o = {group // 2}; o > 0; o >>= 1) {{")
                self.indent += 1
                self._line(f"const {cty} other = __shfl_xor_sync({member_mask}, {part}[g], o);")
                self._line(f"{part}[g] = {self._combine(op.opcode, element, f'{part}[g]', 'other')};")
                self.indent -= 1
                self._line("}")
                self.indent -= 1
                self._line("}")
            name = f"v{tag}_{lay.index}_0"
            self._stmt(lay, f"{cty} {name}[{lay.regs}];", f"{name}[r] = {part}[r / {lay.vec}];")
            row_totals = _Inst("array", name)
            self.inst[(result.id, broadcast_ctx)] = row_totals
            wanted = [ctx for ctx in wanted if ctx != broadcast_ctx]
            if not wanted:
                return
            # another use: one shared slot per row, written by the row's first vector slot
            slots = f"rowred_{tag}"
            self.shared_lines.append(f"    __shared__ {cty} {slots}[{rows}];")
            self._flush()
            self._line("#pragma unroll")
            self._line(f"for (int g = 0; g < {groups}; ++g) {{")
            self.indent += 1
            first = f"L{lay.index}[g * {lay.vec}]"
            in_shape = f"{first} < {lay.numel} && " if lay.guarded else ""
            self._line(f"if ({in_shape}{first} % {cols} == 0) {slots}[{first} / {cols}] = {part}[g];")
            self.indent -= 1
            self._line("}")
            self._line("__syncthreads();")
            read_row = lambda row: f"{slots}[{row}]"                       # noqa: E731
        else:
            # general geometry: one shared slot per vector, combined per row by whoever needs it
            slots = f"rowred_{tag}"
            per_row = group
            if rows * per_row * 4 > 48 * 1024:
                raise TypeError(f"axis reduction of a {rows}x{cols} block needs more than 48 KiB of shared memory")
            self.shared_lines.append(f"    __shared__ {cty} {slots}[{rows * per_row}];")
            self._line("#pragma unroll")
            self._line(f"for (int g = 0; g < {groups}; ++g) {{")
            self.indent += 1
            first = f"L{lay.index}[g * {lay.vec}]"
            guard = f"if ({first} < {lay.numel}) " if lay.guarded else ""
            self._line(f"{guard}{slots}[{first} / {lay.vec}] = {part}[g];")
            self.indent -= 1
            self._line("}")
            self._line("__syncthreads();")

            def read_row(row: str) -> str:
                terms = f"{slots}[({row}) * {per_row}]"
                for g in range(1, per_row):
                    terms = self._combine(op.opcode, element, terms, f"{slots}[({row}) * {per_row} + {g}]")
                return terms

        for ctx in wanted:
            target = self._layout(ctx.shape)
            name = f"v{tag}_{target.index}_" + "".join(map(str, ctx.amap))
            row = self._coord(target, ctx.amap[0], "r")
            valid = self._valid(target, "r")
            row = f"({valid} ? {row} : 0)" if valid else row
            self._stmt(target, f"{cty} {name}[{target.regs}];", f"{name}[r] = {read_row(row)};")
            self.inst[(result.id, ctx)] = _Inst("array", name)
        self._flush()
        if self.loop_depth:
            self._line("__syncthreads();")      # the slots are rewritten by the next iteration

    def _emit_column_reduction(self, op: SSAOp) -> None:
        """``tl.sum/max/min(x, axis=0)``: one value per column.  A column's elements are spread
        over threads and registers with no regular pattern, so the tile goes through shared
        memory once (at most 48 KiB) and every consumer slot walks down its column — adjacent
        lanes read adjacent columns, so the walk is free of bank conflicts."""
        operand, result = op.operands[0], op.result
        assert isinstance(operand, SSAValue) and result is not None
        rows, cols = operand.ty.shape
        element = operand.ty.element
        if (op.opcode, element) not in _IDENTITY:
            raise TypeError(f"Unsupported type for {op.opcode}: {element}")
        if rows * cols * 4 > 48 * 1024:
            raise TypeError(f"axis=0 reduction of a {rows}x{cols} block needs more than 48 KiB of shared memory")
        identity, cty = _IDENTITY[(op.opcode, element)], self.cuda_type(element)
        own = self._own_ctx(operand.ty)
        lay = self._layout(own.shape)
        source = self._get(operand, own)
        tile = f"coltile_{result.id}"
        self.shared_lines.append(f"    __shared__ {cty} {tile}[{rows * cols}];")
        valid = self._valid(lay, "r")
        write = f"{tile}[L{lay.index}[r]] = {source.at('r')};"
        self._stmt(lay, None, f"if {valid} {{ {write} }}" if valid else write)
        self._flush()
        self._line("__syncthreads();")
        for ctx in self.demand.get(result.id, []):
            target = self._layout(ctx.shape)
            name = f"v{result.id}_{target.index}_" + "".join(map(str, ctx.amap))
            column = self._coord(target, ctx.amap[0], "r")
            guard = self._valid(target, "r")
            column = f"({guard} ? {column} : 0)" if guard else column
            self._flush()
            self._line(f"{cty} {name}[{target.regs}];")
            self._line("#pragma unroll")
            self._line(f"for (int r = 0; r < {target.regs}; ++r) {{")
            self.indent += 1
            self._line(f"const int column = {column};")
            self._line(f"{cty} acc = {identity};")
            self._line(f"for (int i = 0; i < {rows}; ++i) acc = "
                       f"{self._combine(op.opcode, element, 'acc', f'{tile}[i * {cols} + column]')};")
            self._line(f"{name}[r] = acc;")
            self.indent -= 1
            self._line("}")
            self.inst[(result.id, ctx)] = _Inst("array", name)
        if self.loop_depth:
            self._line("__syncthreads();")      # the tile is rewritten by the next iteration

    def _emit_cta_combine(self, opcode: str, element: ScalarType, cty: str, part: str,
                          name: str, tag: str) -> None:
        """CTA-wide combine of one per-thread partial; the result lands in every thread."""
        threads = self.threads
        if threads == 1:
            self._line(f"{cty} {name} = {part};")
            return
        pow2 = threads & (threads - 1) == 0
        if threads < 32 and not pow2:
            slots = f"red_{tag}"
            self.shared_lines.append(f"    __shared__ {cty} {slots}[{threads}];")
            self._line(f"{slots}[threadIdx.x] = {part};")
            self._line("__syncthreads();")
            self._line(f"{cty} {name} = {slots}[0];")
            self._line(f"for (int w = 1; w < {threads}; ++w) {name} = {self._combine(opcode, element, name, f'{slots}[w]')};")
            if self.loop_depth:
                self._line("__syncthreads();")
            return
        width = min(threads, 32)
        member_mask = "0xffffffffu" if width == 32 else hex((1 << width) - 1) + "u"
        self._line("#pragma unroll")
        self._line(f"for (int o = {width // 2}; o > 0; o >>= 1) {{")
        self.indent += 1
        # the exchange gets its own statement: a ternary combine would otherwise evaluate
        # the shuffle a second time inside a divergent branch
        self._line(f"const {cty} other = __shfl_xor_sync({member_mask}, {part}, o);")
        self._line(f"{part} = {self._combine(opcode, element, part, 'other')};")
        self.indent -= 1
        self._line("}")
        if threads <= 32:
            self._line(f"{cty} {name} = {part};")
            return
        warps = threads // 32
        slots = f"red_{tag}"
        self.shared_lines.append(f"    __shared__ {cty} {slots}[{warps}];")
        self._line(f"if ((threadIdx.x & 31) == 0) {slots}[threadIdx.x >> 5] = {part};")
        self._line("__syncthreads();")
        self._line(f"{cty} {name} = {slots}[0];")
        self._line("#pragma unroll")
        self._line(f"for (int w = 1; w < {warps}; ++w) {name} = {self._combine(opcode, element, name, f'{slots}[w]')};")
        if self.loop_depth:
            self._line("__syncthreads();")

    # ------------------------------------------------------------------ emission: online softmax

    def _match_online_softmax(self, ops: list[SSAItem], position: int):
        """ops[position] is `m = max(x)`; look for d = x - m; e = exp(d); s = sum(e)
        with m, d used nowhere else.  Returns (sub, exp, sum) ops or None."""
        first = ops[position]
        if not isinstance(first, SSAOp) or first.opcode != "max":
            return None
        if element_of(first.operands[0].ty) != F32:
            return None
        x, m = first.operands[0], first.result
        tail = [op for op in ops[position + 1:]]
        if any(isinstance(op, SSAForRange) for op in tail[:3]) or len(tail) < 3:
            return None
        sub, exp, total = tail[0], tail[1], tail[2]
        ok = (
            sub.opcode == "sub" and sub.operands == (x, m)
            and exp.opcode == "exp" and exp.operands == (sub.result,)
            and total.opcode == "sum" and total.operands == (exp.result,)
        )
        if not ok:
            return None
        uses_m = uses_d = 0
        for op in self._walk(ops):
            for operand in getattr(op, "operands", ()):
                uses_m += operand == m
                uses_d += operand == sub.result
        return (sub, exp, total) if uses_m == 1 and uses_d == 1 else None

    def _walk(self, ops):
        for op in ops:
            if isinstance(op, SSAForRange):
                yield from self._walk(op.body)
            else:
                yield op

    def _emit_online_softmax(self, first: SSAOp, sub: SSAOp, exp: SSAOp, total: SSAOp) -> None:
        """One pass over the thread's registers keeps a running (max, sum) pair; the
        pairs are merged across the CTA with a single exchange.  exp(x - max) for the
        numerators is then evaluated once with the final max, as in the two-reduction
        form, so the stored quotient uses the same operations per element."""
        x = first.operands[0]
        ctx = self._own_ctx(x.ty)
        lay = self._layout(ctx.shape)
        source = self._get(x, ctx)
        self._flush()
        neg_inf = _IDENTITY[("max", F32)]
        rid = first.result.id
        m, s = f"om{rid}", f"os{rid}"

        def lane(r: str) -> str:
            valid = self._valid(lay, r)
            return f"({valid} ? {source.at(r)} : {neg_inf})" if valid else source.at(r)

        self._line(f"float {m} = {lane('0')};")
        if lay.regs > 1:
            self._line("#pragma unroll")
            self._line(f"for (int r = 1; r < {lay.regs}; ++r) {m} = fmaxf({m}, {lane('r')});")
        self._line(f"float {s} = 0.0f;")
        self._line("#pragma unroll")
        safe = f"({m} == {neg_inf} ? 0.0f : {m})"
        self._line(f"for (int r = 0; r < {lay.regs}; ++r) {s} += expf({lane('r')} - {safe});")
        threads = self.threads
        if threads > 1:
            width = min(threads, 32)
            member_mask = "0xffffffffu" if width == 32 else hex((1 << width) - 1) + "u"
            self._line("#pragma unroll")
            self._line(f"for (int o = {width // 2}; o > 0; o >>= 1) {{")
            self.indent += 1
            self._line(f"const float m2 = __shfl_xor_sync({member_mask}, {m}, o);")
            self._line(f"const float s2 = __shfl_xor_sync({member_mask}, {s}, o);")
            self._line(f"const float mm = fmaxf({m}, m2);")
            self._line(f"const float ms = (mm == {neg_inf} ? 0.0f : mm);")
            self._line(f"{s} = {s} * expf({m} - ms) + s2 * expf(m2 - ms);")
            self._line(f"{m} = mm;")
            self.indent -= 1
            self._line("}")
        if threads > 32:
            warps = threads // 32
            self.shared_lines.append(f"    __shared__ float2 osm_{rid}[{warps}];")
            self._line(f"if ((threadIdx.x & 31) == 0) osm_{rid}[threadIdx.x >> 5] = make_float2({m}, {s});")
            self._line("__syncthreads();")
            self._line(f"{m} = osm_{rid}[0].x;")
            self._line("#pragma unroll")
            self._line(f"for (int w = 1; w < {warps}; ++w) {m} = fmaxf({m}, osm_{rid}[w].x);")
            self._line(f"const float osafe{rid} = ({m} == {neg_inf} ? 0.0f : {m});")
            self._line(f"{s} = 0.0f;")
            self._line("#pragma unroll")
            self._line(f"for (int w = 0; w < {warps}; ++w) {s} += osm_{rid}[w].y * expf(osm_{rid}[w].x - osafe{rid});")
            if self.loop_depth:
                self._line("__syncthreads();")
        self._line(f"const float v{first.result.id} = {m};")
        self._line(f"const float v{total.result.id} = {s};")
        self.inst[(first.result.id, None)] = _Inst("scalar", f"v{first.result.id}")
        self.inst[(total.result.id, None)] = _Inst("scalar", f"v{total.result.id}")
        # numerators, for whoever consumes them (normally the final division)
        for follow in (sub, exp):
            for follow_ctx in self.demand.get(follow.result.id, []):
                self._emit_block(follow, follow_ctx)

    # ------------------------------------------------------------------ emission: SIMT dot

    def _emit_dot(self, op: SSAOp) -> None:
        result = op.result
        assert result is not None and isinstance(result.ty, BlockType)
        a_op, b_op, acc_op = op.operands
        a_ty, b_ty = self._type_of(a_op), self._type_of(b_op)
        bm, bk = a_ty.shape
        bn = b_ty.shape[1]
        staging = (bm * bk + bk * bn) * 4
        if staging > 200 * 1024:
            raise TypeError(
                f"tl.dot tile {bm}x{bn}x{bk} needs more than 200 KiB of staging on the SIMT "
                "path; use the K-loop form that lowers to tcgen05"
            )
        a = self._get(a_op, self._own_ctx(a_ty))
        b = self._get(b_op, self._own_ctx(b_ty))
        lay_a, lay_b = self._layout(a_ty.shape), self._layout(b_ty.shape)
        lay_c = self._layout(result.ty.shape)
        acc = self._get(acc_op, self._own_ctx(result.ty)) if acc_op is not None else None
        self._flush()
        sa, sb = f"dot_a_{result.id}", f"dot_b_{result.id}"
        if staging > 32 * 1024:
            # past the static limit the two tiles live in dynamic shared memory; every dot
            # ends with a barrier after its last read, so all of them can share the region
            if not self.dynamic_smem:
                self.shared_lines.append("    extern __shared__ float mtb_dot_staging[];")
            self.dynamic_smem = max(self.dynamic_smem, staging)
            self.shared_lines.append(f"    float* const {sa} = mtb_dot_staging;")
            self.shared_lines.append(f"    float* const {sb} = mtb_dot_staging + {bm * bk};")
        else:
            self.shared_lines.append(f"    __shared__ float {sa}[{bm * bk}];")
            self.shared_lines.append(f"    __shared__ float {sb}[{bk * bn}];")
        for lay, inst, smem in ((lay_a, a, sa), (lay_b, b, sb)):
            self._line("#pragma unroll")
            self._line(f"for (int r = 0; r < {lay.regs}; ++r) {{")
            valid = self._valid(lay, "r")
            write = f"{smem}[L{lay.index}[r]] = {inst.at('r')};"
            self._line("    " + (f"if {valid} {{ {write} }}" if valid else write))
            self._line("}")
        self._line("__syncthreads();")
        name = f"v{result.id}_{lay_c.index}"
        self._line(f"float {name}[{lay_c.regs}];")
        self._line("#pragma unroll")
        self._line(f"for (int r = 0; r < {lay_c.regs}; ++r) {{")
        self.indent += 1
        self._line(f"float sum = {acc.at('r') if acc else '0.0f'};")
        valid = self._valid(lay_c, "r")

        def clamped(coordinate: str) -> str:      # slots outside the tile read element 0
            return f"({valid} ? {coordinate} : 0)" if valid else coordinate

        self._line(f"const int ci = {clamped(self._coord(lay_c, 0, 'r'))};")
        self._line(f"const int cj = {clamped(self._coord(lay_c, 1, 'r'))};")
        self._line(f"for (int k = 0; k < {bk}; ++k) sum = fmaf({sa}[ci * {bk} + k], {sb}[k * {bn} + cj], sum);")
        self._line(f"{name}[r] = sum;")
        self.indent -= 1
        self._line("}")
        self._line("__syncthreads();")
        self.inst[(result.id, self._own_ctx(result.ty))] = _Inst("array", name)
        self._emit_redistribution(result)

    # ------------------------------------------------------------------ emission: loops

    def _emit_for_range(self, loop: SSAForRange) -> None:
        self._flush()
        start = self._get(loop.start, None).text
        stop = self._get(loop.stop, None).text
        step = self._get(loop.step, None).text
        slots: list[tuple[SSAValue, _Inst, _Layout | None]] = []
        for initial, arg, result in zip(loop.carried_inputs, loop.carried_args, loop.results, strict=True):
            pointer = isinstance(element_of(result.ty), PointerType)
            cty = "int" if pointer else self.cuda_type(result.ty)     # a carried pointer is its i32 offset
            if pointer:
                ctx = self._own_ctx(result.ty) if isinstance(result.ty, BlockType) else None
                source = self._get(initial, ctx)
                lay = self._layout(ctx.shape) if ctx is not None else None
                name = f"v{result.id}_{lay.index}" if lay is not None else f"v{result.id}"
                start_at = (lambda r: source.index.at(r)) if source.index is not None else (lambda r: "0")
                if lay is not None:
                    self._stmt(lay, f"int {name}[{lay.regs}];", f"{name}[r] = {start_at('r')};")
                    offset = _Inst("array", name)
                else:
                    self._flush()
                    self._line(f"int {name} = {start_at('r')};")
                    offset = _Inst("scalar", name)
                inst = _Inst("ptr", base=source.base, index=offset, elem=source.elem)
                self.inst[(arg.id, ctx)] = inst
                self.inst[(result.id, ctx)] = inst
                slots.append((result, inst, lay))
                continue
            if isinstance(result.ty, BlockType):
                ctx = self._own_ctx(result.ty)
                lay = self._layout(ctx.shape)
                name = f"v{result.id}_{lay.index}"
                source = self._get(initial, ctx) if isinstance(self._type_of(initial), BlockType) \
                    else self._get(initial, None)
                self._stmt(lay, f"{cty} {name}[{lay.regs}];", f"{name}[r] = {source.at('r')};")
                inst = _Inst("array", name)
                self.inst[(arg.id, ctx)] = inst
                self.inst[(result.id, ctx)] = inst
                slots.append((result, inst, lay))
            else:
                name = f"v{result.id}"
                self._flush()
                self._line(f"{cty} {name} = {self._get(initial, None).text};")
                inst = _Inst("scalar", name)
                self.inst[(arg.id, None)] = inst
                self.inst[(result.id, None)] = inst
                slots.append((result, inst, None))
        self._flush()
        index = f"v{loop.index.id}"
        self.inst[(loop.index.id, None)] = _Inst("scalar", index)
        self._line(f"for (int {index} = {start}; {index} < {stop}; {index} += {step}) {{")
        self.indent += 1
        self.loop_depth += 1
        for arg in loop.carried_args:
            self._emit_redistribution(arg)      # per iteration: the carried value changes
        self._emit_ops(loop.body)
        self._flush()
        # yields: stage through temporaries when a yield reads another carried slot
        carried_ids = {arg.id for arg in loop.carried_args}
        staged = any(isinstance(y, SSAValue) and y.id in carried_ids for y in loop.yields)
        moves: list[tuple[_Inst, _Inst, _Layout | None, str]] = []
        for yielded, (result, inst, lay) in zip(loop.yields, slots, strict=True):
            if inst.kind == "ptr":
                ctx = self._own_ctx(result.ty) if lay is not None else None
                advanced = self._get(yielded, ctx)
                if advanced.base != inst.base:
                    raise TypeError("a loop-carried pointer must keep pointing into the same array")
                if advanced.index is None:
                    raise TypeError("a loop-carried pointer lost its offset")
                moves.append((inst.index, advanced.index, lay, "int"))
                continue
            if lay is not None:
                src = self._get(yielded, self._own_ctx(result.ty)) \
                    if isinstance(self._type_of(yielded), BlockType) else self._get(yielded, None)
            else:
                src = self._get(yielded, None)
            moves.append((inst, src, lay, self.cuda_type(result.ty)))
        if staged:
            temps = []
            for target, src, lay, cty in moves:
                temp = self._fresh("carry")
                if lay is None:
                    self._line(f"const {cty} {temp} = {src.text};")
                    temps.append(_Inst("scalar", temp))
                else:
                    self._stmt(lay, f"{cty} {temp}[{lay.regs}];", f"{temp}[r] = {src.at('r')};")
                    temps.append(_Inst("array", temp))
            self._flush()
            moves = [(target, temp, lay, cty) for (target, _, lay, cty), temp in zip(moves, temps)]
        for target, src, lay, _ in moves:
            if lay is None:
                self._flush()
                self._line(f"{target.text} = {src.text};")
            else:
                self._stmt(lay, None, f"{target.text}[r] = {src.at('r')};")
        self._flush()
        self.loop_depth -= 1
        self.indent -= 1
        self._line("}")
        for result in loop.results:
            self._emit_redistribution(result)

    # ------------------------------------------------------------------ driver

    def _emit_ops(self, ops: list[SSAItem]) -> None:
        skip: set[int] = set()
        for position, op in enumerate(ops):
            if id(op) in skip:
                continue
            if isinstance(op, SSAForRange):
                self._emit_for_range(op)
                continue
            if op.opcode in ("store", "atomic_add"):
                self._emit_store(op)
                continue
            if op.opcode == "break_unless":
                # the condition is a program-uniform scalar, so every thread of the CTA
                # leaves together and barriers later in the body stay safe
                self._flush()
                self._line(f"if (!({self._get(op.operands[0], None).text})) break;")
                continue
            if op.opcode in ("sum", "max", "min") and "axis" in op.attrs:
                self._emit_axis_reduction(op)
                continue
            if op.opcode in ("sum", "max", "min"):
                fused = self._match_online_softmax(ops, position) if self.online_softmax else None
                if fused is not None:
                    self._emit_online_softmax(op, *fused)
                    skip.update(id(x) for x in fused)
                else:
                    self._emit_reduction(op)
                continue
            if op.opcode == "dot":
                self._emit_dot(op)
                continue
            if op.opcode not in self.ELEMENTWISE and op.opcode not in ("program_id", "num_programs", "expand_dims", "trans"):
                raise TypeError(f"Unsupported SSA opcode: {op.opcode}")
            result = op.result
            if result is None:
                raise TypeError(f"SSA opcode {op.opcode!r} requires a result")
            if isinstance(result.ty, BlockType):
                for ctx in self.demand.get(result.id, []):
                    self._emit_block(op, ctx)
            else:
                self._emit_scalar(op)

    def generate_artifact(self, kernel_name: str, ssa_ops: list[SSAItem], params: list[Param]) -> KernelArtifact:
        from . import dot_codegen  # local import: dot_codegen imports this module

        self._reset()
        cuda_kernel_block_shape_check(ssa_ops)
        matched = dot_codegen.match_gemm_loop(ssa_ops, params) if self.tensor_cores else None
        if matched is not None:
            return dot_codegen.generate_gemm(kernel_name, matched, params, self)

        self.param_positions = {param.name: position for position, param in enumerate(params)}
        self._index_ops(ssa_ops)
        self._analyse_affine(ssa_ops)
        self._analyse_demand(ssa_ops)
        self.threads = self._choose_threads()
        for contexts in self.demand.values():      # all layout prologues go first
            for ctx in contexts:
                self._layout(ctx.shape)
        self._emit_ops(ssa_ops)
        self._flush()

        signature = ", ".join(f"{self.cuda_type(p.ty)} {p.name}" for p in params)
        text = []
        checked_arrays = [p.name for p in params if isinstance(p.ty, PointerType)] if self.bounds_check else []
        if self.bounds_check:
            # the arrays' extents (in elements) and the status word follow the kernel's own parameters
            signature += "".join(f", long long mtb_ext_{name}" for name in checked_arrays) + ", unsigned* mtb_oob"
            text += [_BOUNDS_HELPERS, ""]
        if self.uses_half_helpers:
            text += [_HALF_HELPERS, ""]
        text += [
            'extern "C" __global__ __launch_bounds__(%s)' % (
                f"{self.threads}, {self.min_ctas_per_sm}" if self.min_ctas_per_sm else self.threads),
            f"void {kernel_name}({signature}) {{",
        ]
        text += self.shared_lines
        if self.shared_lines:
            text.append("")
        text += self.lines
        text.append("}")
        plan = LaunchPlan(kernel_name=kernel_name, threads=self.threads, dynamic_smem=self.dynamic_smem)
        if self.bounds_check:
            plan.notes["bounds_check"] = checked_arrays
        plan.notes["layouts"] = {
            "x".join(map(str, lay.shape)): {"regs": lay.regs, "vec": lay.vec}
            for lay in self.layouts.values()
        }
        return KernelArtifact("\n".join(text), plan)

    def generate(self, kernel_name: str, ssa_ops: list[SSAItem], params: list[Param]) -> str:
        return self.generate_artifact(kernel_name, ssa_ops, params).src


def cuda_kernel_block_shape_check(ssa_ops: list[SSAItem]) -> None:
    """Keep the reference's diagnostics for kernels it rejects on shape grounds
    (more than one vector width in a rank-1 kernel; rank > 2), except that kernels
    using ``tl.dot`` legitimately mix tile shapes."""

    def has_dot(ops) -> bool:
        for op in ops:
            if isinstance(op, SSAForRange):
                if has_dot(op.body):
                    return True
            elif op.opcode in ("dot", "trans"):       # tiles of more than one shape are their business
                return True
        return False

    if not has_dot(ssa_ops):
        cuda_kernel_block_shape(ssa_ops)
