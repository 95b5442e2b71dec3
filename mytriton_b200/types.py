"""Type objects of the kernel language.

The three type families and their printed forms (``i32``, ``ptr<f32>``,
``vector<8 x f32>``, ``block<4x8 x f32>``) follow the reference's
``src/mytriton/trace.py:166-236`` because the typed-SSA text is part of the
public contract.  ``bf16`` and ``ptr<bf16>`` are additions needed by ``tl.dot``.
"""

from __future__ import annotations

from dataclasses import dataclass
from math import prod


@dataclass(frozen=True)
class ScalarType:
    name: str

    def __str__(self) -> str:
        return self.name


@dataclass(frozen=True)
class PointerType:
    element: ScalarType
    address_space: str = "global"

    def __str__(self) -> str:
        inner = str(self.element)
        if self.address_space != "global":
            inner = f"{self.address_space}, {inner}"
        return f"ptr<{inner}>"


@dataclass(frozen=True)
class BlockType:
    shape: tuple[int, ...]
    element: ScalarType | PointerType

    def __post_init__(self) -> None:
        if len(self.shape) == 0:
            raise TypeError("block shape must not be empty")
        if min(self.shape) <= 0:
            raise TypeError(f"block dimensions must be positive, got {self.shape}")

    @property
    def rank(self) -> int:
        return len(self.shape)

    @property
    def num_elements(self) -> int:
        return prod(self.shape)

    @property
    def size(self) -> int:
        if len(self.shape) != 1:
            raise TypeError(f"rank-{self.rank} block has no single size")
        return self.shape[0]

    def __str__(self) -> str:
        if len(self.shape) == 1:
            return f"vector<{self.shape[0]} x {self.element}>"
        dims = "x".join(map(str, self.shape))
        return f"block<{dims} x {self.element}>"


def VectorType(size: int, element: ScalarType | PointerType) -> BlockType:
    return BlockType((size,), element)


Type = ScalarType | PointerType | BlockType

I32 = ScalarType("i32")
F32 = ScalarType("f32")
BOOL = ScalarType("bool")
BF16 = ScalarType("bf16")
F16 = ScalarType("f16")
F8E4M3 = ScalarType("f8e4m3")      # 8-bit float, 4 exponent / 3 mantissa bits, no infinities
PTR_F32 = PointerType(F32)
PTR_BF16 = PointerType(BF16)
PTR_F16 = PointerType(F16)
F8E5M2 = ScalarType("f8e5m2")      # 8-bit float, 5 exponent / 2 mantissa bits (the top byte of fp16)
PTR_F8E4M3 = PointerType(F8E4M3)
PTR_F8E5M2 = PointerType(F8E5M2)

# names the ``tl`` namespace exposes
int1 = BOOL
int32 = I32
float32 = F32
bfloat16 = BF16
float16 = F16
float8e4nv = F8E4M3
float8e5 = F8E5M2

NUMERIC = (I32, F32, BF16, F16, F8E4M3, F8E5M2)
FLOATING = (F32, BF16, F16, F8E4M3, F8E5M2)
HALF_WIDTH = (BF16, F16)      # 16-bit storage types; values are widened to fp32 in registers
BYTE_WIDTH = (F8E4M3, F8E5M2)        # 8-bit storage types, widened likewise


# f32 -> f32 functions of the language besides ``exp`` (which the reference has): the SSA opcode
# is the name, the CUDA spelling is the value.
FLOAT_UNARY = {
    "sqrt": "sqrtf", "rsqrt": "rsqrtf", "log": "logf", "log2": "log2f", "exp2": "exp2f",
    "sin": "sinf", "cos": "cosf", "tanh": "tanhf", "abs": "fabsf",
    # x.to(tl.float16) / x.to(tl.bfloat16): the value rounded to that precision (to nearest even);
    # registers hold fp32 throughout, 16-bit types exist in memory only
    "round_f16": "mtb_round_f16", "round_bf16": "mtb_round_bf16",
}


def element_of(ty: Type) -> ScalarType | PointerType:
    return ty.element if isinstance(ty, BlockType) else ty


def shape_of(ty: Type) -> tuple[int, ...]:
    return ty.shape if isinstance(ty, BlockType) else ()
