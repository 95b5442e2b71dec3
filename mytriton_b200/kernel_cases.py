"""Compile cases shared by the golden-fixture generator and the tests.

Each case names a corpus kernel, its runtime arguments (arrays are given by
shape; their contents never matter for compilation), its constexpr values and a
launch grid.  ``expect_error`` marks kernels that must be rejected.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import numpy as np


@dataclass(frozen=True)
class Case:
    name: str
    kernel: str
    args: tuple[Any, ...]            # ("f32", shape) for arrays, or Python scalars
    constexprs: dict[str, Any] = field(default_factory=dict)
    grid: tuple[int, ...] = (1,)
    expect_error: str | None = None  # exception class name


def A(*shape: int) -> tuple[str, tuple[int, ...]]:
    return ("f32", tuple(shape))


def build_args(case: Case) -> list[Any]:
    return [
        np.zeros(arg[1], dtype=np.float32) if isinstance(arg, tuple) and arg and arg[0] == "f32"
        else arg
        for arg in case.args
    ]


CASES: list[Case] = [
    Case("add_1024", "add_kernel", (A(98432), A(98432), A(98432), 98432), {"BLOCK": 1024}, (97,)),
    Case("add_256", "add_kernel", (A(1000), A(1000), A(1000), 1000), {"BLOCK": 256}, (4,)),
    Case("copy_256", "copy_kernel", (A(1000), A(1000), 1000), {"BLOCK": 256}, (4,)),
    Case("relu_256", "relu_kernel", (A(1000), A(1000), 1000), {"BLOCK": 256}, (4,)),
    Case("relu_1024", "relu_kernel", (A(5000), A(5000), 5000), {"BLOCK": 1024}, (5,)),
    Case("leaky_relu_256", "leaky_relu_kernel", (A(1000), A(1000), 1000, 0.01), {"BLOCK": 256}, (4,)),
    Case("leaky_relu_1024", "leaky_relu_kernel", (A(5000), A(5000), 5000, 0.01), {"BLOCK": 1024}, (5,)),
    Case("sigmoid_256", "sigmoid_kernel", (A(1000), A(1000), 1000), {"BLOCK": 256}, (4,)),
    Case("sigmoid_1024", "sigmoid_kernel", (A(5000), A(5000), 5000), {"BLOCK": 1024}, (5,)),
    Case("row_sum_1024", "row_sum_kernel", (A(127, 513), A(127), 513), {"BLOCK": 1024}, (127,)),
    Case("row_sum_8", "row_sum_kernel", (A(3, 5), A(3), 5), {"BLOCK": 8}, (3,)),
    Case("row_max_1024", "row_max_kernel", (A(127, 513), A(127), 513), {"BLOCK": 1024}, (127,)),
    Case("row_min_1024", "row_min_kernel", (A(127, 513), A(127), 513), {"BLOCK": 1024}, (127,)),
    Case("softmax_1024", "softmax_kernel", (A(127, 513), A(127, 513), 513), {"BLOCK": 1024}, (127,)),
    Case("softmax_8", "softmax_kernel", (A(3, 5), A(3, 5), 5), {"BLOCK": 8}, (3,)),
    Case("softmax_1", "softmax_kernel", (A(4, 1), A(4, 1), 1), {"BLOCK": 1}, (4,)),
    Case("softmax_4096", "softmax_kernel", (A(8, 4096), A(8, 4096), 4096), {"BLOCK": 4096}, (8,),
         ),
    Case("long_row_sum_static", "long_row_sum_kernel", (A(31, 4097), A(31)),
         {"N_COLS": 4097, "BLOCK": 256}, (31,)),
    Case("long_row_sum_loop_1024", "long_row_sum_loop_kernel", (A(31, 4097), A(31), 4097),
         {"BLOCK": 1024}, (31,)),
    Case("matrix_add_256", "matrix_add_kernel", (A(127, 513), A(127, 513), A(127, 513), 513),
         {"BLOCK": 256}, (127, 3)),
    Case("tile_shape_4x8", "tile_shape_kernel", (A(3, 5), 3, 5), {"BM": 4, "BN": 8}, (1,)),
    Case("matrix_add_2d_16x32", "matrix_add_2d_kernel", (A(127, 513), A(127, 513), A(127, 513), 127, 513),
         {"BM": 16, "BN": 32}, (8, 17)),
    Case("unparenthesized_mask", "invalid_unparenthesized_mask_kernel", (A(4, 8), A(4, 8), 4, 8),
         {"BM": 4, "BN": 8}, (1,), expect_error="TypeError"),
    Case("naive_matmul_k17", "naive_matmul_kernel", (A(31, 17), A(17, 513), A(31, 513), 513),
         {"K": 17, "BLOCK": 256}, (31, 3)),
    Case("matmul_2d_k5", "matmul_2d_kernel", (A(19, 5), A(5, 23), A(19, 23), 19, 23),
         {"K": 5, "BM": 8, "BN": 16}, (3, 2)),
    Case("matmul_runtime_k", "matmul_runtime_k_kernel", (A(19, 5), A(5, 23), A(19, 23), 19, 23, 5),
         {"BM": 8, "BN": 16}, (3, 2)),
    Case("matmul_runtime_k_4x8", "matmul_runtime_k_kernel", (A(5, 3), A(3, 7), A(5, 7), 5, 7, 3),
         {"BM": 4, "BN": 8}, (2, 1)),
    Case("matmul_runtime_k_32x32", "matmul_runtime_k_kernel", (A(64, 64), A(64, 64), A(64, 64), 64, 64, 64),
         {"BM": 32, "BN": 32}, (2, 2)),
    Case("two_carried", "two_carried_values_kernel", (A(1), 4)),
    Case("annotated_carried", "annotated_carried_value_kernel", (A(1), 3)),
    Case("no_carried", "no_carried_values_kernel", (A(3), 3)),
    Case("sequential_loops", "sequential_runtime_loops_kernel", (A(1), 3)),
    Case("nested_loops", "nested_runtime_loops_kernel", (A(1), 4)),
    Case("bad_step_0", "invalid_runtime_step_kernel", (A(1), 3), {"STEP": 0}, expect_error="ASTFrontendError"),
    Case("bad_step_neg", "invalid_runtime_step_kernel", (A(1), 3), {"STEP": -1}, expect_error="ASTFrontendError"),
    Case("assigned_induction", "assigned_induction_variable_kernel", (A(1), 3), expect_error="ASTFrontendError"),
    Case("full_and_zeros", "full_and_zeros_kernel", (A(5), 5), {"BLOCK": 8}),
    Case("runtime_full_int", "runtime_full_kernel", (A(5), 5, 3), {"BLOCK": 8}),
    Case("runtime_full_float", "runtime_full_kernel", (A(5), 5, 1.25), {"BLOCK": 8}),
    Case("empty_block", "empty_kernel", (A(5), 5), {"BLOCK": 8}),
    Case("inconsistent_width", "inconsistent_width_kernel", (A(256), 256), expect_error="ValueError"),
    Case("tile_32", "tile_kernel", (A(32), 32), {"TILE_SIZE": 32}),
    Case("scalar_copy", "scalar_copy_kernel", (A(1), A(1))),
    Case("nested_pointer", "nested_pointer_kernel", (A(4),)),
    Case("nonzero_range", "nonzero_range_kernel", (A(8),)),
    Case("compile_only", "compile_only_kernel", (A(16), A(16), A(16), 16), {"TILE": 16}),
    Case("extremum", "extremum_kernel", (2.0, 3.0, A(1), A(1))),
    Case("int_reduce_64", "int_reduce_kernel", (A(80), 37), {"BLOCK": 64}),
    Case("int_reduce_1024", "int_reduce_kernel", (A(1100), 700), {"BLOCK": 1024}),
    Case("matrix_add_2d_6x10", "matrix_add_2d_kernel", (A(13, 27), A(13, 27), A(13, 27), 13, 27),
         {"BM": 6, "BN": 10}, (3, 3)),
    Case("tile_shape_3x5", "tile_shape_kernel", (A(3, 5), 3, 5), {"BM": 3, "BN": 5}, (1,)),
    Case("softmax_64", "softmax_kernel", (A(9, 50), A(9, 50), 50), {"BLOCK": 64}, (9,)),
    Case("row_sum_2", "row_sum_kernel", (A(5, 2), A(5), 2), {"BLOCK": 2}, (5,)),
    Case("add_48", "add_kernel", (A(100), A(100), A(100), 100), {"BLOCK": 48}, (3,)),
    Case("chunked_row_stats_256", "chunked_row_stats_kernel", (A(17, 1000), A(17), A(17), 1000),
         {"BLOCK": 256}, (17,)),
    Case("where_minimum_256", "where_minimum_kernel", (A(1000), A(1000), A(1000), 1000), {"BLOCK": 256}, (4,)),
]

CASES_BY_NAME = {case.name: case for case in CASES}
