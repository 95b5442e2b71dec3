"""The kernel corpus: every program the backend must accept unchanged.

The first group restates, kernel for kernel, the ``@triton.jit`` functions of
the reference's test-suite (file:line given at each kernel) — they define what
"drop-in" means.  The second group holds the kernels the benchmark
configurations add (runtime-loop long-row sum, bf16 ``tl.dot`` matmul).

The module can be bound to either implementation: by default to
``mytriton_b200``; with ``CORPUS_IMPL=reference`` (used only by
tests/golden/make_golden.py, in a container where the reference is importable)
to the reference package, so that both compile the very same source text.
"""

from __future__ import annotations

import os
from typing import Any

if os.environ.get("CORPUS_IMPL") == "reference":
    import mytriton as triton
    import mytriton.language as tl
else:
    import mytriton_b200 as triton
    import mytriton_b200.language as tl


# ---------------------------------------------------------------- rank-1 elementwise

@triton.jit
def add_kernel(x, y, out, n, BLOCK: tl.constexpr):  # tests/test_add_kernel.py:25-35
    pid = tl.program_id(0)
    offs = pid * BLOCK + tl.arange(0, BLOCK)
    mask = offs < n
    a = tl.load(x + offs, mask=mask, other=0.0)
    b = tl.load(y + offs, mask=mask, other=0.0)
    tl.store(out + offs, a + b, mask=mask)


@triton.jit
def copy_kernel(x, out, n, BLOCK: tl.constexpr):  # tests/test_copy_kernel.py:25-34
    pid = tl.program_id(0)
    offs = pid * BLOCK + tl.arange(0, BLOCK)
    mask = offs < n
    values = tl.load(x + offs, mask=mask, other=0.0)
    tl.store(out + offs, values, mask=mask)


@triton.jit
def relu_kernel(x, out, n, BLOCK: tl.constexpr):  # tests/test_relu_kernel.py:12-21
    pid = tl.program_id(0)
    offs = pid * BLOCK + tl.arange(0, BLOCK)
    mask = offs < n
    a = tl.load(x + offs, mask=mask, other=0.0)
    tl.store(out + offs, tl.maximum(a, 0.0), mask=mask)


@triton.jit
def leaky_relu_kernel(x, out, n, alpha, BLOCK: tl.constexpr):  # tests/test_leaky_relu_kernel.py:12-23
    pid = tl.program_id(0)
    offs = pid * BLOCK + tl.arange(0, BLOCK)
    mask = offs < n
    a = tl.load(x + offs, mask=mask, other=0.0)
    result = tl.where(a < 0.0, alpha * a, a)
    tl.store(out + offs, result, mask=mask)


@triton.jit
def sigmoid_kernel(x, out, n, BLOCK: tl.constexpr):  # tests/test_sigmoid_kernel.py:12-23
    pid = tl.program_id(0)
    offs = pid * BLOCK + tl.arange(0, BLOCK)
    mask = offs < n
    a = tl.load(x + offs, mask=mask, other=0.0)
    result = 1.0 / (1.0 + tl.exp(-a))
    tl.store(out + offs, result, mask=mask)


# ---------------------------------------------------------------- row reductions, softmax

@triton.jit
def row_sum_kernel(x, out, n_cols, BLOCK: tl.constexpr):  # tests/test_reduce_sum_kernel.py:27-41
    row = tl.program_id(0)
    cols = tl.arange(0, BLOCK)
    offsets = row * n_cols + cols
    mask = cols < n_cols
    values = tl.load(x + offsets, mask=mask, other=0.0)
    total = tl.sum(values)
    first_lane = cols < 1
    tl.store(out + row, total, mask=first_lane)


@triton.jit
def row_max_kernel(x, out, n_cols, BLOCK: tl.constexpr):  # tests/test_reduce_extremum_kernel.py:13-27
    row = tl.program_id(0)
    cols = tl.arange(0, BLOCK)
    offsets = row * n_cols + cols
    mask = cols < n_cols
    values = tl.load(x + offsets, mask=mask, other=float("-inf"))
    result = tl.max(values)
    first_lane = cols < 1
    tl.store(out + row, result, mask=first_lane)


@triton.jit
def row_min_kernel(x, out, n_cols, BLOCK: tl.constexpr):  # tests/test_reduce_extremum_kernel.py:30-44
    row = tl.program_id(0)
    cols = tl.arange(0, BLOCK)
    offsets = row * n_cols + cols
    mask = cols < n_cols
    values = tl.load(x + offsets, mask=mask, other=float("inf"))
    result = tl.min(values)
    first_lane = cols < 1
    tl.store(out + row, result, mask=first_lane)


@triton.jit
def softmax_kernel(x, out, n_cols, BLOCK: tl.constexpr):  # tests/test_softmax_kernel.py:29-47
    row = tl.program_id(0)
    cols = tl.arange(0, BLOCK)
    offsets = row * n_cols + cols
    mask = cols < n_cols
    values = tl.load(x + offsets, mask=mask, other=float("-inf"))
    row_max = tl.max(values)
    numerators = tl.exp(values - row_max)
    denominator = tl.sum(numerators)
    probabilities = numerators / denominator
    tl.store(out + offsets, probabilities, mask=mask)


@triton.jit
def long_row_sum_kernel(x, out, N_COLS: tl.constexpr, BLOCK: tl.constexpr):  # tests/test_long_row_sum_kernel.py:28-47
    row = tl.program_id(0)
    lanes = tl.arange(0, BLOCK)
    row_start = row * N_COLS
    partial: Any = 0.0
    for start in tl.static_range(0, N_COLS, BLOCK):
        cols = start + lanes
        mask = cols < N_COLS
        values = tl.load(x + row_start + cols, mask=mask, other=0.0)
        partial = partial + values
    total = tl.sum(partial)
    first_lane = lanes < 1
    tl.store(out + row, total, mask=first_lane)


# ---------------------------------------------------------------- 2-D grids and tiles

@triton.jit
def matrix_add_kernel(x, y, out, n_cols, BLOCK: tl.constexpr):  # tests/test_matrix_add_kernel.py:24-37
    row = tl.program_id(0)
    col_block = tl.program_id(1)
    cols = col_block * BLOCK + tl.arange(0, BLOCK)
    offsets = row * n_cols + cols
    mask = cols < n_cols
    lhs = tl.load(x + offsets, mask=mask, other=0.0)
    rhs = tl.load(y + offsets, mask=mask, other=0.0)
    tl.store(out + offsets, lhs + rhs, mask=mask)


@triton.jit
def tile_shape_kernel(out, M, N, BM: tl.constexpr, BN: tl.constexpr):  # tests/test_tile_shape_kernel.py:15-22
    offs_m = tl.arange(0, BM)[:, None]
    offs_n = tl.arange(0, BN)[None, :]
    offsets = offs_m * N + offs_n
    mask = (offs_m < M) & (offs_n < N)
    tl.store(out + offsets, offsets, mask=mask)


@triton.jit
def matrix_add_2d_kernel(x, y, out, M, N, BM: tl.constexpr, BN: tl.constexpr):  # tests/test_tile_shape_kernel.py:61-75
    pid_m = tl.program_id(0)
    pid_n = tl.program_id(1)
    offs_m = pid_m * BM + tl.arange(0, BM)[:, None]
    offs_n = pid_n * BN + tl.arange(0, BN)[None, :]
    offsets = offs_m * N + offs_n
    mask = (offs_m < M) & (offs_n < N)
    lhs = tl.load(x + offsets, mask=mask, other=0.0)
    rhs = tl.load(y + offsets, mask=mask, other=0.0)
    tl.store(out + offsets, lhs + rhs, mask=mask)


@triton.jit
def invalid_unparenthesized_mask_kernel(x, out, M, N, BM: tl.constexpr, BN: tl.constexpr):  # tests/test_tile_shape_kernel.py:78-93
    offs_m = tl.arange(0, BM)[:, None]
    offs_n = tl.arange(0, BN)[None, :]
    mask = offs_m < M & offs_n < N
    offsets = offs_m * N + offs_n
    tl.store(out + offsets, tl.load(x + offsets, mask=mask), mask=mask)


# ---------------------------------------------------------------- SIMT matmuls

@triton.jit
def naive_matmul_kernel(a, b, c, n_cols, K: tl.constexpr, BLOCK: tl.constexpr):  # tests/test_naive_matmul_kernel.py:27-57
    row = tl.program_id(0)
    col_block = tl.program_id(1)
    cols = col_block * BLOCK + tl.arange(0, BLOCK)
    mask = cols < n_cols
    accumulator: Any = 0.0
    a_row_start = row * K
    for k in tl.static_range(0, K):
        a_value = tl.load(a + a_row_start + k)
        b_offsets = k * n_cols + cols
        b_values = tl.load(b + b_offsets, mask=mask, other=0.0)
        accumulator = accumulator + a_value * b_values
    c_offsets = row * n_cols + cols
    tl.store(c + c_offsets, accumulator, mask=mask)


@triton.jit
def matmul_2d_kernel(a, b, c, M, N, K: tl.constexpr, BM: tl.constexpr, BN: tl.constexpr):  # tests/test_matmul_2d_kernel.py:11-45
    pid_m = tl.program_id(0)
    pid_n = tl.program_id(1)
    offs_m = pid_m * BM + tl.arange(0, BM)[:, None]
    offs_n = pid_n * BN + tl.arange(0, BN)[None, :]
    c_offsets = offs_m * N + offs_n
    c_mask = (offs_m < M) & (offs_n < N)
    acc = tl.zeros((BM, BN), tl.float32)
    for k in tl.static_range(0, K):
        a_offsets = offs_m * K + k
        b_offsets = k * N + offs_n
        a_mask = offs_m < M
        b_mask = offs_n < N
        a_values = tl.load(a + a_offsets, mask=a_mask, other=0.0)
        b_values = tl.load(b + b_offsets, mask=b_mask, other=0.0)
        acc = acc + a_values * b_values
    tl.store(c + c_offsets, acc, mask=c_mask)


@triton.jit
def matmul_runtime_k_kernel(a, b, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr):  # tests/test_ast_runtime_loop.py:22-53
    pid_m = tl.program_id(0)
    pid_n = tl.program_id(1)
    offs_m = pid_m * BM + tl.arange(0, BM)[:, None]
    offs_n = pid_n * BN + tl.arange(0, BN)[None, :]
    c_offsets = offs_m * N + offs_n
    c_mask = (offs_m < M) & (offs_n < N)
    acc = tl.zeros((BM, BN), tl.float32)
    for k in range(K):
        a_offsets = offs_m * K + k
        b_offsets = k * N + offs_n
        a_values = tl.load(a + a_offsets, mask=offs_m < M, other=0.0)
        b_values = tl.load(b + b_offsets, mask=offs_n < N, other=0.0)
        acc = acc + a_values * b_values
    tl.store(c + c_offsets, acc, mask=c_mask)


# ---------------------------------------------------------------- scalar runtime loops

@triton.jit
def two_carried_values_kernel(out, n):  # tests/test_ast_runtime_loop.py:56-65
    first = 0
    second = 1
    for k in range(n):
        first = first + k
        second = second + first
    tl.store(out, first + second)


@triton.jit
def annotated_carried_value_kernel(out, n):  # tests/test_ast_runtime_loop.py:68-75
    acc: Any = 0
    for k in range(n):
        acc: Any = acc + k  # type: ignore[no-redef]
    tl.store(out, acc)


@triton.jit
def no_carried_values_kernel(out, n):  # tests/test_ast_runtime_loop.py:78-81
    for k in range(n):
        tl.store(out + k, k)


@triton.jit
def sequential_runtime_loops_kernel(out, n):  # tests/test_ast_runtime_loop.py:84-93
    acc = 0
    for i in range(n):
        acc = acc + i
    for j in range(n):
        acc = acc + j
    tl.store(out, acc)


@triton.jit
def nested_runtime_loops_kernel(out, n):  # tests/test_ast_runtime_loop.py:96-104
    offset = tl.program_id(0)
    acc: Any = 0
    for i in range(n):
        for j in range(n):
            acc = acc + offset + i + j
    tl.store(out + offset, acc)


@triton.jit
def invalid_runtime_step_kernel(out, n, STEP: tl.constexpr):  # tests/test_ast_runtime_loop.py:107-113
    acc = 0
    for k in range(0, n, STEP):
        acc = acc + k
    tl.store(out, acc)


@triton.jit
def assigned_induction_variable_kernel(out, n):  # tests/test_ast_runtime_loop.py:116-121
    for k in range(n):
        k += 1
    tl.store(out, 0.0)


# ---------------------------------------------------------------- constructors and small probes

@triton.jit
def full_and_zeros_kernel(out, n, BLOCK: tl.constexpr):  # tests/test_block_constructors.py:11-17
    offsets = tl.arange(0, BLOCK)
    mask = offsets < n
    values = tl.zeros((BLOCK,), tl.float32)
    values = values + tl.full([BLOCK], 2.5, tl.float32)
    tl.store(out + offsets, values, mask=mask)


@triton.jit
def runtime_full_kernel(out, n, value, BLOCK: tl.constexpr):  # tests/test_block_constructors.py:20-25
    offsets = tl.arange(0, BLOCK)
    mask = offsets < n
    values = tl.full(BLOCK, value, tl.float32)
    tl.store(out + offsets, values, mask=mask)


@triton.jit
def empty_kernel(out, n, BLOCK: tl.constexpr):  # tests/test_block_constructors.py:28-33
    offsets = tl.arange(0, BLOCK)
    mask = offsets < n
    values = tl.empty((BLOCK,), tl.float32)
    tl.store(out + offsets, values, mask=mask)


@triton.jit
def inconsistent_width_kernel(out, n):  # tests/test_cuda_compiler.py:13-18
    short_offsets = tl.arange(0, 128)
    long_offsets = tl.arange(0, 256)
    tl.store(out + short_offsets, 1.0, mask=short_offsets < n)
    tl.store(out + long_offsets, 2.0, mask=long_offsets < n)


@triton.jit
def tile_kernel(out, n, TILE_SIZE: tl.constexpr):  # tests/test_cuda_compiler.py:21-24
    offsets = tl.program_id(0) * TILE_SIZE + tl.arange(0, TILE_SIZE)
    tl.store(out + offsets, 1.0, mask=offsets < n)


@triton.jit
def scalar_copy_kernel(source, out):  # tests/test_cuda_compiler.py:27-30
    value = tl.load(source)
    tl.store(out, value)


@triton.jit
def nested_pointer_kernel(out):  # tests/test_cuda_compiler.py:33-35
    tl.store(out + 1 + 2, 1.0)


@triton.jit
def nonzero_range_kernel(out):  # tests/test_cuda_compiler.py:38-41
    offsets = tl.arange(4, 8)
    tl.store(out + offsets, 1.0)


@triton.jit
def compile_only_kernel(x, y, out, n, TILE: tl.constexpr):  # tests/test_cuda_compiler.py:44-50
    offsets = tl.arange(0, TILE)
    mask = offsets < n
    x_values = tl.load(x + offsets, mask=mask)
    y_values = tl.load(y + offsets, mask=mask)
    tl.store(out + offsets, x_values + y_values, mask=mask)


@triton.jit
def extremum_kernel(lhs, rhs, out_max, out_min):
    """Scalar form of the reference's extremum execution cases
    (tests/test_math_ops.py:253-291), as a kernel instead of hand-built SSA."""
    tl.store(out_max, tl.maximum(lhs, rhs))
    tl.store(out_min, tl.minimum(lhs, rhs))


@triton.jit
def int_reduce_kernel(out, n, BLOCK: tl.constexpr):
    """i32 reductions and i32 arithmetic (C division truncates toward zero:
    src/mytriton/cuda_codegen.py:37-44); results are stored into an f32 array."""
    lanes = tl.arange(0, BLOCK)
    values = (lanes - n) * 3 / 2
    first = lanes < 1
    tl.store(out + 0, tl.sum(values), mask=first)
    tl.store(out + 1, tl.max(values), mask=first)
    tl.store(out + 2, tl.min(values), mask=first)
    tl.store(out + 3 + lanes, values / 4 - -values, mask=lanes < n)


@triton.jit
def where_minimum_kernel(x, y, out, n, BLOCK: tl.constexpr):
    """tl.where with mixed i32/f32 arms, tl.minimum on blocks, & of masks, negation."""
    pid = tl.program_id(0)
    offs = pid * BLOCK + tl.arange(0, BLOCK)
    mask = (offs < n) & (offs < n + 1)
    a = tl.load(x + offs, mask=mask, other=1.5)
    b = tl.load(y + offs, mask=mask)
    picked = tl.where(a < b, offs, -b)
    tl.store(out + offs, tl.minimum(picked, a) + tl.maximum(a, b), mask=mask)


@triton.jit
def chunked_row_stats_kernel(x, out_max, out_sum, n_cols, BLOCK: tl.constexpr):
    """Reductions inside a runtime loop with scalar loop-carried values: the running
    maximum and the running sum of a row, one BLOCK-wide chunk at a time."""
    row = tl.program_id(0)
    lanes = tl.arange(0, BLOCK)
    running_max = float("-inf")
    running_sum = 0.0
    for start in range(0, n_cols, BLOCK):
        cols = start + lanes
        mask = cols < n_cols
        values = tl.load(x + row * n_cols + cols, mask=mask, other=float("-inf"))
        running_max = tl.maximum(running_max, tl.max(values))
        running_sum = running_sum + tl.sum(tl.where(mask, values, 0.0))
    first = lanes < 1
    tl.store(out_max + row, running_max, mask=first)
    tl.store(out_sum + row, running_sum, mask=first)


# ---------------------------------------------------------------- benchmark-config kernels
# (kernels below this line use only features the reference also accepts, unless noted)

@triton.jit
def long_row_sum_loop_kernel(x, out, n_cols, BLOCK: tl.constexpr):
    """Runtime-loop long-row sum: one program streams a whole row.  The reference
    compiles this form too (loop-carried ``vector<BLOCK x f32>``, BLOCK <= 1024)."""
    row = tl.program_id(0)
    lanes = tl.arange(0, BLOCK)
    row_start = row * n_cols
    partial = tl.zeros((BLOCK,), tl.float32)
    for start in range(0, n_cols, BLOCK):
        cols = start + lanes
        mask = cols < n_cols
        values = tl.load(x + row_start + cols, mask=mask, other=0.0)
        partial = partial + values
    total = tl.sum(partial)
    first_lane = lanes < 1
    tl.store(out + row, total, mask=first_lane)


if os.environ.get("CORPUS_IMPL") != "reference":

    @triton.jit
    def matmul_dot_kernel(a, b, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
        """Tiled matmul through ``tl.dot`` (new surface: the reference has no dot and
        accepts only float32 arrays).  a[M,K], b[K,N] row-major (bf16, fp16 or fp8 e4m3
        arrays); c[M,N] fp32."""
        pid_m = tl.program_id(0)
        pid_n = tl.program_id(1)
        offs_m = pid_m * BM + tl.arange(0, BM)
        offs_n = pid_n * BN + tl.arange(0, BN)
        acc = tl.zeros((BM, BN), tl.float32)
        for k0 in range(0, K, BK):
            offs_k = k0 + tl.arange(0, BK)
            a_mask = (offs_m[:, None] < M) & (offs_k[None, :] < K)
            b_mask = (offs_k[:, None] < K) & (offs_n[None, :] < N)
            a_tile = tl.load(a + offs_m[:, None] * K + offs_k[None, :], mask=a_mask, other=0.0)
            b_tile = tl.load(b + offs_k[:, None] * N + offs_n[None, :], mask=b_mask, other=0.0)
            acc = tl.dot(a_tile, b_tile, acc)
        c_mask = (offs_m[:, None] < M) & (offs_n[None, :] < N)
        tl.store(c + offs_m[:, None] * N + offs_n[None, :], acc, mask=c_mask)

    @triton.jit
    def tile_softmax_kernel(x, out, stats, n_rows, n_cols, BM: tl.constexpr, BN: tl.constexpr):
        """Softmax over the rows of a [BM, BN] tile (BM short rows per program), with reductions
        along the tile's last axis: the row maxima and sums are broadcast back over the tile,
        and also stored as vectors (row sum of exponentials, row maximum)."""
        rows = tl.program_id(0) * BM + tl.arange(0, BM)
        cols = tl.arange(0, BN)
        mask = (rows[:, None] < n_rows) & (cols[None, :] < n_cols)
        v = tl.load(x + rows[:, None] * n_cols + cols[None, :], mask=mask, other=float("-inf"))
        peak = tl.max(v, axis=1)
        e = tl.exp(v - peak[:, None])
        total = tl.sum(e, axis=1)
        tl.store(out + rows[:, None] * n_cols + cols[None, :], e / total[:, None], mask=mask)
        tl.store(stats + rows * 2, total, mask=rows < n_rows)
        tl.store(stats + rows * 2 + 1, peak, mask=rows < n_rows)

    @triton.jit
    def attention_kernel(q, k, v, out, seq, scale, BM: tl.constexpr, BN: tl.constexpr, D: tl.constexpr):
        """softmax(q k^T * scale) v for one head in the streaming ("flash") form: per block of BM
        queries a running row maximum, a running normaliser and an unnormalised accumulator are
        carried over blocks of BN keys.  q, k, v, out: [seq, D] row-major fp32.  Exercises row
        reductions of a tile, carried vectors broadcast over tiles, and tl.dot on a computed
        operand."""
        offs_m = tl.program_id(0) * BM + tl.arange(0, BM)
        offs_d = tl.arange(0, D)
        q_tile = tl.load(q + offs_m[:, None] * D + offs_d[None, :], mask=offs_m[:, None] < seq, other=0.0)
        m_i = tl.full((BM,), float("-inf"), tl.float32)
        l_i = tl.zeros((BM,), tl.float32)
        acc = tl.zeros((BM, D), tl.float32)
        for start in range(0, seq, BN):
            offs_n = start + tl.arange(0, BN)
            k_t = tl.load(k + offs_n[None, :] * D + offs_d[:, None], mask=offs_n[None, :] < seq, other=0.0)
            s = tl.dot(q_tile, k_t) * scale
            s = tl.where(offs_n[None, :] < seq, s, float("-inf"))
            m_new = tl.maximum(m_i, tl.max(s, axis=1))
            alpha = tl.exp(m_i - m_new)
            p = tl.exp(s - m_new[:, None])
            l_i = l_i * alpha + tl.sum(p, axis=1)
            v_tile = tl.load(v + offs_n[:, None] * D + offs_d[None, :], mask=offs_n[:, None] < seq, other=0.0)
            acc = acc * alpha[:, None] + tl.dot(p, v_tile)
            m_i = m_new
        tl.store(out + offs_m[:, None] * D + offs_d[None, :], acc / l_i[:, None], mask=offs_m[:, None] < seq)

    @triton.jit
    def layer_norm_kernel(x, weight, bias, out, n_cols, eps, BLOCK: tl.constexpr):
        """Row-wise layer normalisation, one program per row, the row held in registers:
        y = (x - mean) * rsqrt(var + eps) * weight + bias.  Uses the f32 functions the
        reference lacks (rsqrt); one read of x, one write of y."""
        row = tl.program_id(0)
        cols = tl.arange(0, BLOCK)
        mask = cols < n_cols
        v = tl.load(x + row * n_cols + cols, mask=mask, other=0.0)
        mean = tl.sum(v) / n_cols
        centred = tl.where(mask, v - mean, 0.0)
        variance = tl.sum(centred * centred) / n_cols
        scale = tl.rsqrt(variance + eps)
        w = tl.load(weight + cols, mask=mask, other=0.0)
        b = tl.load(bias + cols, mask=mask, other=0.0)
        tl.store(out + row * n_cols + cols, centred * scale * w + b, mask=mask)

    @triton.jit
    def matmul_pointer_bump_kernel(a, b, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
        """The K-loop in its other common spelling: blocks of pointers carried through the loop
        and advanced each iteration, masks written against the remaining depth ``K - k0``, and
        ``acc += tl.dot(...)``."""
        offs_m = tl.program_id(0) * BM + tl.arange(0, BM)
        offs_n = tl.program_id(1) * BN + tl.arange(0, BN)
        offs_k = tl.arange(0, BK)
        a_ptrs = a + offs_m[:, None] * K + offs_k[None, :]
        b_ptrs = b + offs_k[:, None] * N + offs_n[None, :]
        acc = tl.zeros((BM, BN), tl.float32)
        for k0 in range(0, K, BK):
            a_tile = tl.load(a_ptrs, mask=(offs_m[:, None] < M) & (offs_k[None, :] < K - k0), other=0.0)
            b_tile = tl.load(b_ptrs, mask=(offs_k[:, None] < K - k0) & (offs_n[None, :] < N), other=0.0)
            acc += tl.dot(a_tile, b_tile)
            a_ptrs += BK
            b_ptrs += BK * N
        tl.store(c + offs_m[:, None] * N + offs_n[None, :], acc,
                 mask=(offs_m[:, None] < M) & (offs_n[None, :] < N))

    @triton.jit
    def matmul_grouped_kernel(a, b, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr,
                              GROUP_M: tl.constexpr):
        """The usual one-axis launch with grouped tile ordering: the program id is split with
        ``//`` and ``%`` into a tile row and a tile column, GROUP_M tile rows at a time."""
        program = tl.program_id(0)
        tiles_n = tl.cdiv(N, BN)
        per_band = GROUP_M * tiles_n                       # programs in one band of GROUP_M tile rows
        band = program // per_band
        band_rows = tl.minimum(tl.cdiv(M, BM) - band * GROUP_M, GROUP_M)     # the last band may be short
        within = program % per_band
        rows = (band * GROUP_M + within % band_rows) * BM + tl.arange(0, BM)
        cols = (within // band_rows) * BN + tl.arange(0, BN)
        kk = tl.arange(0, BK)
        acc = tl.zeros((BM, BN), tl.float32)
        for k0 in range(0, K, BK):
            x = tl.load(a + rows[:, None] * K + (k0 + kk)[None, :],
                        mask=(rows[:, None] < M) & ((k0 + kk)[None, :] < K), other=0.0)
            y = tl.load(b + (k0 + kk)[:, None] * N + cols[None, :],
                        mask=((k0 + kk)[:, None] < K) & (cols[None, :] < N), other=0.0)
            acc = tl.dot(x, y, acc)
        tl.store(c + rows[:, None] * N + cols[None, :], acc, mask=(rows[:, None] < M) & (cols[None, :] < N))

    @triton.jit
    def matmul_guarded_transposed_kernel(a, b, ct, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
        """One-axis launch with ``//`` and ``%`` tile coordinates, an early ``return`` for programs
        past the last tile row, and the result stored as its transpose: ct[N, M] = (a @ b).T."""
        pid = tl.program_id(0)
        num_pid_n = tl.cdiv(N, BN)
        pid_m = pid // num_pid_n
        pid_n = pid % num_pid_n
        if pid_m * BM >= M:
            return
        rows = pid_m * BM + tl.arange(0, BM)
        cols = pid_n * BN + tl.arange(0, BN)
        kk = tl.arange(0, BK)
        acc = tl.zeros((BM, BN), tl.float32)
        for k0 in range(0, K, BK):
            x = tl.load(a + rows[:, None] * K + (k0 + kk)[None, :],
                        mask=(rows[:, None] < M) & ((k0 + kk)[None, :] < K), other=0.0)
            y = tl.load(b + (k0 + kk)[:, None] * N + cols[None, :],
                        mask=((k0 + kk)[:, None] < K) & (cols[None, :] < N), other=0.0)
            acc = tl.dot(x, y, acc)
        tl.store(ct + cols[None, :] * M + rows[:, None], acc, mask=(rows[:, None] < M) & (cols[None, :] < N))

    @triton.jit
    def matmul_causal_kernel(a, b, c, M, N, K, shift,
                             BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
        """tl.dot with an index-dependent epilogue: entries above the ``shift``-th diagonal
        become ``-inf`` (an attention-style causal mask), the others are scaled by 1/(1 + row)."""
        pid_m = tl.program_id(0)
        pid_n = tl.program_id(1)
        offs_m = pid_m * BM + tl.arange(0, BM)
        offs_n = pid_n * BN + tl.arange(0, BN)
        acc = tl.zeros((BM, BN), tl.float32)
        for k0 in range(0, K, BK):
            offs_k = k0 + tl.arange(0, BK)
            a_mask = (offs_m[:, None] < M) & (offs_k[None, :] < K)
            b_mask = (offs_k[:, None] < K) & (offs_n[None, :] < N)
            a_tile = tl.load(a + offs_m[:, None] * K + offs_k[None, :], mask=a_mask, other=0.0)
            b_tile = tl.load(b + offs_k[:, None] * N + offs_n[None, :], mask=b_mask, other=0.0)
            acc = tl.dot(a_tile, b_tile, acc)
        rows = offs_m[:, None]
        cols = offs_n[None, :]
        y = tl.where(rows + shift < cols, float("-inf"), acc / (rows + 1))
        c_mask = (offs_m[:, None] < M) & (offs_n[None, :] < N)
        tl.store(c + offs_m[:, None] * N + offs_n[None, :], y, mask=c_mask)

    @triton.jit
    def branchy_kernel(x, out, n, threshold, BLOCK: tl.constexpr):
        """Run-time ``if``/``else``, ``not`` and an early ``return`` on program-uniform
        scalars (the reference rejects all three).  Programs past the end of the data leave
        first; programs below ``threshold`` double their values, the others negate them and
        add their block sum; ``late`` exists only because both paths bind it."""
        pid = tl.program_id(0)
        offs = pid * BLOCK + tl.arange(0, BLOCK)
        mask = offs < n
        if n - 1 < pid * BLOCK:
            return
        v = tl.load(x + offs, mask=mask, other=0.0)
        if pid < threshold:
            v = v * 2.0
            late = 1.0
        else:
            v = -v
            late = tl.sum(v)
        if not (pid < 2):
            v = v + late
        tl.store(out + offs, v, mask=mask)

    @triton.jit
    def branch_in_loop_kernel(x, out, n_cols, skip, BLOCK: tl.constexpr):
        """A run-time ``if`` inside a run-time loop, with loads and a carried value under
        it, and a loop inside a run-time ``if``: row ``r`` sums every chunk except chunk
        number ``skip``; odd rows then add the row's first chunk once more."""
        row = tl.program_id(0)
        lanes = tl.arange(0, BLOCK)
        acc = tl.zeros((BLOCK,), tl.float32)
        chunk = 0
        for start in range(0, n_cols, BLOCK):
            cols = start + lanes
            if chunk < skip:
                acc = acc + tl.load(x + row * n_cols + cols, mask=cols < n_cols, other=0.0)
            else:
                if skip < chunk:
                    acc = acc + tl.load(x + row * n_cols + cols, mask=cols < n_cols, other=0.0)
            chunk = chunk + 1
        parity = row - (row / 2) * 2
        if parity > 0:
            for start in range(0, BLOCK, BLOCK):
                cols = start + lanes
                acc = acc + tl.load(x + row * n_cols + cols, mask=cols < n_cols, other=0.0)
        tl.store(out + row, tl.sum(acc))

    @triton.jit
    def collatz_kernel(out, limit):
        """``while`` on a run-time scalar, with an ``if``/``else`` in its body: the number of
        Collatz steps from ``pid + 1`` down to 1, at most ``limit``."""
        pid = tl.program_id(0)
        value = pid + 1
        steps = 0
        while (1 < value) & (steps < limit):
            half = value / 2
            if value - half * 2 > 0:
                value = value * 3 + 1
            else:
                value = half
            steps = steps + 1
        tl.store(out + pid, steps)

    @triton.jit
    def while_chunks_kernel(x, out, n_cols, budget, BLOCK: tl.constexpr):
        """``while`` whose condition depends on a block reduction made in its body: a row is
        summed chunk by chunk until the running sum of magnitudes passes ``budget`` (or the
        row ends); the row's sum so far and the number of columns consumed are stored."""
        row = tl.program_id(0)
        lanes = tl.arange(0, BLOCK)
        acc = tl.zeros((BLOCK,), tl.float32)
        start = 0
        spent = 0.0
        while (start < n_cols) & (spent < budget):
            cols = start + lanes
            v = tl.load(x + row * n_cols + cols, mask=cols < n_cols, other=0.0)
            acc = acc + v
            spent = spent + tl.sum(tl.where(v < 0.0, -v, v))
            start = start + BLOCK
        tl.store(out + row * 2, tl.sum(acc))
        tl.store(out + row * 2 + 1, start)

    @triton.jit
    def matmul_nt_kernel(a, bt, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
        """C = A @ Bt.T with Bt stored [N, K] row-major (a weight matrix as frameworks keep it):
        the [BK, BN] tile of B is read through the transposed index expression."""
        offs_m = tl.program_id(0) * BM + tl.arange(0, BM)
        offs_n = tl.program_id(1) * BN + tl.arange(0, BN)
        acc = tl.zeros((BM, BN), tl.float32)
        for k0 in range(0, K, BK):
            offs_k = k0 + tl.arange(0, BK)
            a_tile = tl.load(a + offs_m[:, None] * K + offs_k[None, :],
                             mask=(offs_m[:, None] < M) & (offs_k[None, :] < K), other=0.0)
            b_tile = tl.load(bt + offs_n[None, :] * K + offs_k[:, None],
                             mask=(offs_k[:, None] < K) & (offs_n[None, :] < N), other=0.0)
            acc = tl.dot(a_tile, b_tile, acc)
        tl.store(c + offs_m[:, None] * N + offs_n[None, :], acc,
                 mask=(offs_m[:, None] < M) & (offs_n[None, :] < N))

    @triton.jit
    def matmul_tn_kernel(at, b, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
        """C = At.T @ B with At stored [K, M] row-major (x.T @ dy, the weight gradient of a linear
        layer): the [BM, BK] tile of A is read through the transposed index expression."""
        offs_m = tl.program_id(0) * BM + tl.arange(0, BM)
        offs_n = tl.program_id(1) * BN + tl.arange(0, BN)
        acc = tl.zeros((BM, BN), tl.float32)
        for k0 in range(0, K, BK):
            offs_k = k0 + tl.arange(0, BK)
            a_tile = tl.load(at + offs_k[None, :] * M + offs_m[:, None],
                             mask=(offs_m[:, None] < M) & (offs_k[None, :] < K), other=0.0)
            b_tile = tl.load(b + offs_k[:, None] * N + offs_n[None, :],
                             mask=(offs_k[:, None] < K) & (offs_n[None, :] < N), other=0.0)
            acc = tl.dot(a_tile, b_tile, acc)
        tl.store(c + offs_m[:, None] * N + offs_n[None, :], acc,
                 mask=(offs_m[:, None] < M) & (offs_n[None, :] < N))

    @triton.jit
    def matmul_tt_kernel(at, bt, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
        """C = At.T @ Bt.T with both operands stored transposed ([K, M] and [N, K])."""
        offs_m = tl.program_id(0) * BM + tl.arange(0, BM)
        offs_n = tl.program_id(1) * BN + tl.arange(0, BN)
        acc = tl.zeros((BM, BN), tl.float32)
        for k0 in range(0, K, BK):
            offs_k = k0 + tl.arange(0, BK)
            a_tile = tl.load(at + offs_k[None, :] * M + offs_m[:, None],
                             mask=(offs_m[:, None] < M) & (offs_k[None, :] < K), other=0.0)
            b_tile = tl.load(bt + offs_n[None, :] * K + offs_k[:, None],
                             mask=(offs_k[:, None] < K) & (offs_n[None, :] < N), other=0.0)
            acc = tl.dot(a_tile, b_tile, acc)
        tl.store(c + offs_m[:, None] * N + offs_n[None, :], acc,
                 mask=(offs_m[:, None] < M) & (offs_n[None, :] < N))

    @triton.jit
    def matmul_strided_kernel(a, b, c, M, N, K, stride_am, stride_ak, stride_bk, stride_bn, stride_cm, stride_cn,
                              BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
        """The matmul as it is usually written, with every stride an argument: which of them is 1
        says how A, B and C are stored, and is known only at the call."""
        offs_m = tl.program_id(0) * BM + tl.arange(0, BM)
        offs_n = tl.program_id(1) * BN + tl.arange(0, BN)
        acc = tl.zeros((BM, BN), tl.float32)
        for k0 in range(0, K, BK):
            offs_k = k0 + tl.arange(0, BK)
            a_tile = tl.load(a + offs_m[:, None] * stride_am + offs_k[None, :] * stride_ak,
                             mask=(offs_m[:, None] < M) & (offs_k[None, :] < K), other=0.0)
            b_tile = tl.load(b + offs_k[:, None] * stride_bk + offs_n[None, :] * stride_bn,
                             mask=(offs_k[:, None] < K) & (offs_n[None, :] < N), other=0.0)
            acc = tl.dot(a_tile, b_tile, acc)
        tl.store(c + offs_m[:, None] * stride_cm + offs_n[None, :] * stride_cn, acc,
                 mask=(offs_m[:, None] < M) & (offs_n[None, :] < N))

    @triton.jit
    def matmul_tutorial_kernel(a, b, c, M, N, K, stride_am, stride_ak, stride_bk, stride_bn, stride_cm, stride_cn,
                               BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr, GROUP_M: tl.constexpr):
        """A matmul the way such kernels are commonly written: a one-axis grid whose programs walk
        the tiles band by band (GROUP_M tile rows at a time, for L2 reuse), every stride an
        argument, blocks of pointers advanced in a loop that counts k-blocks, masks against the
        depth that is left, ``acc = tl.dot(a, b, acc)``."""
        program = tl.program_id(0)
        tiles_m = tl.cdiv(M, BM)
        tiles_n = tl.cdiv(N, BN)
        per_band = GROUP_M * tiles_n
        band = program // per_band
        band_rows = tl.minimum(tiles_m - band * GROUP_M, GROUP_M)
        within = program % per_band
        tile_m = band * GROUP_M + within % band_rows
        tile_n = within // band_rows
        rows = tile_m * BM + tl.arange(0, BM)
        cols = tile_n * BN + tl.arange(0, BN)
        depth = tl.arange(0, BK)
        a_block = a + (rows[:, None] * stride_am + depth[None, :] * stride_ak)
        b_block = b + (depth[:, None] * stride_bk + cols[None, :] * stride_bn)
        acc = tl.zeros((BM, BN), tl.float32)
        for step in range(0, tl.cdiv(K, BK)):
            left = K - step * BK
            a_tile = tl.load(a_block, mask=(rows[:, None] < M) & (depth[None, :] < left), other=0.0)
            b_tile = tl.load(b_block, mask=(depth[:, None] < left) & (cols[None, :] < N), other=0.0)
            acc = tl.dot(a_tile, b_tile, acc)
            a_block += BK * stride_ak
            b_block += BK * stride_bk
        tl.store(c + stride_cm * rows[:, None] + stride_cn * cols[None, :], acc,
                 mask=(rows[:, None] < M) & (cols[None, :] < N))

    @triton.jit
    def matmul_tutorial_modulo_kernel(a, b, c, M, N, K, stride_am, stride_ak, stride_bk, stride_bn, stride_cm,
                                      stride_cn, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr,
                                      GROUP_M: tl.constexpr):
        """``matmul_tutorial_kernel`` with the operands' row and column indices taken modulo M and N
        instead of masked (rows past the edge read rows from the top; the store's mask drops them)."""
        program = tl.program_id(0)
        tiles_m = tl.cdiv(M, BM)
        tiles_n = tl.cdiv(N, BN)
        per_band = GROUP_M * tiles_n
        band = program // per_band
        band_rows = tl.minimum(tiles_m - band * GROUP_M, GROUP_M)
        within = program % per_band
        tile_m = band * GROUP_M + within % band_rows
        tile_n = within // band_rows
        rows = tile_m * BM + tl.arange(0, BM)
        cols = tile_n * BN + tl.arange(0, BN)
        depth = tl.arange(0, BK)
        a_block = a + ((rows % M)[:, None] * stride_am + depth[None, :] * stride_ak)
        b_block = b + (depth[:, None] * stride_bk + (cols % N)[None, :] * stride_bn)
        acc = tl.zeros((BM, BN), tl.float32)
        for step in range(0, tl.cdiv(K, BK)):
            left = K - step * BK
            a_tile = tl.load(a_block, mask=depth[None, :] < left, other=0.0)
            b_tile = tl.load(b_block, mask=depth[:, None] < left, other=0.0)
            acc = tl.dot(a_tile, b_tile, acc)
            a_block += BK * stride_ak
            b_block += BK * stride_bk
        tl.store(c + stride_cm * rows[:, None] + stride_cn * cols[None, :], acc,
                 mask=(rows[:, None] < M) & (cols[None, :] < N))

    @triton.jit
    def linear_layer_kernel(x, w, y, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
        """y = x @ w.T with the weight [N, K] as frameworks keep it: a [BN, BK] tile of w is loaded as
        it lies in memory and transposed in the call, ``tl.dot(x_tile, tl.trans(w_tile), acc)``."""
        rows = tl.program_id(0) * BM + tl.arange(0, BM)
        outs = tl.program_id(1) * BN + tl.arange(0, BN)
        acc = tl.zeros((BM, BN), tl.float32)
        for k0 in range(0, K, BK):
            ks = k0 + tl.arange(0, BK)
            x_tile = tl.load(x + rows[:, None] * K + ks[None, :], mask=(rows[:, None] < M) & (ks[None, :] < K), other=0.0)
            w_tile = tl.load(w + outs[:, None] * K + ks[None, :], mask=(outs[:, None] < N) & (ks[None, :] < K), other=0.0)
            acc = tl.dot(x_tile, tl.trans(w_tile), acc)
        tl.store(y + rows[:, None] * N + outs[None, :], acc, mask=(rows[:, None] < M) & (outs[None, :] < N))

    @triton.jit
    def matmul_residual_kernel(a, b, residual, c, M, N, K, alpha, BM: tl.constexpr, BN: tl.constexpr,
                               BK: tl.constexpr):
        """c = alpha * (a @ b) + residual: the epilogue reads a whole tile of another [M, N] matrix at
        the element's own position (a skip connection; with residual = c, ``c += alpha * a @ b``)."""
        rows = tl.program_id(0) * BM + tl.arange(0, BM)
        cols = tl.program_id(1) * BN + tl.arange(0, BN)
        inside = (rows[:, None] < M) & (cols[None, :] < N)
        acc = tl.zeros((BM, BN), tl.float32)
        for k0 in range(0, K, BK):
            ks = k0 + tl.arange(0, BK)
            acc = tl.dot(tl.load(a + rows[:, None] * K + ks[None, :], mask=(rows[:, None] < M) & (ks[None, :] < K), other=0.0),
                         tl.load(b + ks[:, None] * N + cols[None, :], mask=(ks[:, None] < K) & (cols[None, :] < N), other=0.0),
                         acc)
        skip = tl.load(residual + rows[:, None] * N + cols[None, :], mask=inside, other=0.0)
        tl.store(c + rows[:, None] * N + cols[None, :], acc * alpha + skip, mask=inside)

    @triton.jit
    def strided_scale_kernel(x, out, n, factor, BLOCK: tl.constexpr):
        """A fixed number of programs strides over any number of blocks (``tl.num_programs``)."""
        pid = tl.program_id(0)
        step = tl.num_programs(0)
        lanes = tl.arange(0, BLOCK)
        for i in range(0, tl.cdiv(tl.cdiv(n, BLOCK) - pid, step)):
            offs = (pid + i * step) * BLOCK + lanes
            tl.store(out + offs, tl.load(x + offs, mask=offs < n, other=0.0) * factor, mask=offs < n)

    @triton.jit
    def scan_until_kernel(x, out, n_cols, limit, BLOCK: tl.constexpr):
        """``continue`` and ``break`` in a run-time loop: a row is added up chunk by chunk from the
        left, chunks whose first element is negative are skipped, and the scan stops at the first
        chunk whose sum exceeds ``limit``.  Stored per row: the total, the chunks visited, and the
        column where the scan stopped (-1 if it reached the end)."""
        row = tl.program_id(0)
        lanes = tl.arange(0, BLOCK)
        total = 0.0
        visited = 0
        stopped_at = -1
        for start in range(0, n_cols, BLOCK):
            visited += 1
            head = tl.load(x + row * n_cols + start)
            if head < 0.0:
                continue
            cols = start + lanes
            chunk = tl.sum(tl.load(x + row * n_cols + cols, mask=cols < n_cols, other=0.0))
            if chunk > limit:
                stopped_at = start
                break
            total += chunk
        tl.store(out + row * 3, total)
        tl.store(out + row * 3 + 1, visited)
        tl.store(out + row * 3 + 2, stopped_at)

    @triton.jit
    def first_negative_kernel(x, out, n):
        """``while True`` left by ``break``, one program per row of ``n`` values: the index of the
        row's first negative value (``n`` if there is none) and the sum of the values before it."""
        row = tl.program_id(0)
        index = 0
        total = 0.0
        while True:
            if not index < n:
                break
            value = tl.load(x + row * n + index)
            if value < 0.0:
                break
            total += value
            index += 1
        tl.store(out + row * 2, total)
        tl.store(out + row * 2 + 1, index)

    @triton.jit
    def nested_break_kernel(x, out, n_rows, n_cols, limit, BLOCK: tl.constexpr):
        """An inner ``break`` leaves only the inner loop; the outer loop uses ``continue`` and an
        unrolled loop over a compile-time range is cut short by a run-time ``break``.  One program:
        for every row, chunks are added until one has a negative sum; rows whose total exceeds
        ``limit`` are not counted."""
        lanes = tl.arange(0, BLOCK)
        counted = 0
        grand = 0.0
        for row in range(0, n_rows):
            total = 0.0
            for start in range(0, n_cols, BLOCK):
                cols = start + lanes
                chunk = tl.sum(tl.load(x + row * n_cols + cols, mask=cols < n_cols, other=0.0))
                if chunk < 0.0:
                    break
                total += chunk
            if total > limit:
                continue
            counted += 1
            grand += total
        firsts = 0.0
        for k in range(4):                     # unrolled while tracing
            value = tl.load(x + k)
            if value < 0.0:
                break
            firsts += value
        tl.store(out, grand)
        tl.store(out + 1, counted)
        tl.store(out + 2, firsts)

    @triton.jit
    def matmul_tf32_kernel(a, b, c, M, N, K, BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
        """The same product on float32 arrays with ``input_precision="tf32"``: operands reach
        the tensor cores with 10-bit mantissas, accumulation stays fp32."""
        pid_m = tl.program_id(0)
        pid_n = tl.program_id(1)
        offs_m = pid_m * BM + tl.arange(0, BM)
        offs_n = pid_n * BN + tl.arange(0, BN)
        acc = tl.zeros((BM, BN), tl.float32)
        for k0 in range(0, K, BK):
            offs_k = k0 + tl.arange(0, BK)
            a_mask = (offs_m[:, None] < M) & (offs_k[None, :] < K)
            b_mask = (offs_k[:, None] < K) & (offs_n[None, :] < N)
            a_tile = tl.load(a + offs_m[:, None] * K + offs_k[None, :], mask=a_mask, other=0.0)
            b_tile = tl.load(b + offs_k[:, None] * N + offs_n[None, :], mask=b_mask, other=0.0)
            acc = tl.dot(a_tile, b_tile, acc, input_precision="tf32")
        c_mask = (offs_m[:, None] < M) & (offs_n[None, :] < N)
        tl.store(c + offs_m[:, None] * N + offs_n[None, :], acc, mask=c_mask)

    @triton.jit
    def matmul_bias_act_kernel(a, b, bias, row_scale, c, M, N, K, slope,
                               BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
        """tl.dot followed by elementwise work on the accumulator: a column bias, a
        per-row scale and a leaky-relu, all applied before the one store of C."""
        pid_m = tl.program_id(0)
        pid_n = tl.program_id(1)
        offs_m = pid_m * BM + tl.arange(0, BM)
        offs_n = pid_n * BN + tl.arange(0, BN)
        acc = tl.zeros((BM, BN), tl.float32)
        for k0 in range(0, K, BK):
            offs_k = k0 + tl.arange(0, BK)
            a_mask = (offs_m[:, None] < M) & (offs_k[None, :] < K)
            b_mask = (offs_k[:, None] < K) & (offs_n[None, :] < N)
            a_tile = tl.load(a + offs_m[:, None] * K + offs_k[None, :], mask=a_mask, other=0.0)
            b_tile = tl.load(b + offs_k[:, None] * N + offs_n[None, :], mask=b_mask, other=0.0)
            acc = tl.dot(a_tile, b_tile, acc)
        bias_values = tl.load(bias + offs_n, mask=offs_n < N, other=0.0)
        scale_values = tl.load(row_scale + offs_m, mask=offs_m < M, other=0.0)
        y = (acc + bias_values[None, :]) * scale_values[:, None]
        y = tl.where(y < 0.0, slope * y, y)
        c_mask = (offs_m[:, None] < M) & (offs_n[None, :] < N)
        tl.store(c + offs_m[:, None] * N + offs_n[None, :], y, mask=c_mask)
