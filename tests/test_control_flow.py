"""Run-time ``if`` / ``else`` / ``not`` / early ``return`` (CPU): the front end lowers them
by predication — masks on the loads and stores of a branch, ``select`` for the names the
branches rebind — so the IR gains only the boolean ``not``.  The oracle's SSA interpreter
runs the lowered kernels against closed-form NumPy results."""

import numpy as np
import pytest

from mytriton_b200 import kernels as corpus
import mytriton_b200 as triton
import mytriton_b200.language as tl
from mytriton_b200.ast_frontend import ASTFrontendError
from mytriton_b200.cuda_utils import NVRTC_OPTIONS
from mytriton_b200.ssa import SSAForRange, SSAPrinter
from oracle import ssa_interp


def branchy_expected(x, n, threshold, block):
    out = np.full_like(x, 7.0)
    for pid in range(-(-len(x) // block)):
        if n - 1 < pid * block:
            continue
        sl = slice(pid * block, min((pid + 1) * block, n))
        v = x[sl].astype(np.float32)
        if pid < threshold:
            v, late = v * np.float32(2.0), np.float32(1.0)
        else:
            v = -v
            late = ssa_interp.tree_sum(np.concatenate([v, np.zeros(block - len(v), np.float32)]))
        if not pid < 2:
            v = v + late
        out[sl] = v
    return out


def branch_in_loop_expected(x, skip, block):
    rows, cols = x.shape
    out = np.zeros(rows, np.float32)
    for r in range(rows):
        acc = np.zeros(block, np.float32)
        for chunk, start in enumerate(range(0, cols, block)):
            if chunk != skip:
                piece = x[r, start:start + block]
                acc[:len(piece)] += piece
        if r % 2:
            piece = x[r, :block]
            acc[:len(piece)] += piece
        out[r] = ssa_interp.tree_sum(acc)
    return out


def all_ops(items):
    for item in items:
        if isinstance(item, SSAForRange):
            yield from all_ops(item.body)
        else:
            yield item


def test_if_else_not_and_return_lower_to_masks_and_selects(runtime_lib):
    rng = np.random.default_rng(0)
    n, block, threshold = 1000, 256, 3
    x = rng.standard_normal(6 * block).astype(np.float32)      # two programs past n: they return
    out = np.full_like(x, 7.0)
    grid = (6,)
    _, ssa_ops, src = corpus.branchy_kernel[grid](x, out, n, threshold, BLOCK=block)
    opcodes = [op.opcode for op in all_ops(ssa_ops)]
    assert "not" in opcodes and "select" in opcodes and not any("if" in code for code in opcodes)
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {"x": x, "out": out, "n": n, "threshold": threshold}, grid)
    np.testing.assert_array_equal(out, branchy_expected(x, n, threshold, block))
    runtime_lib.Module(src, "branchy_kernel", NVRTC_OPTIONS)


@pytest.mark.parametrize("skip", [0, 2, 9])
def test_if_inside_a_runtime_loop_and_loop_inside_an_if(skip, runtime_lib):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((5, 700)).astype(np.float32)
    out = np.zeros(5, np.float32)
    _, ssa_ops, src = corpus.branch_in_loop_kernel[(5,)](x, out, 700, skip, BLOCK=256)
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {"x": x, "out": out, "n_cols": 700, "skip": skip}, (5,))
    np.testing.assert_allclose(out, branch_in_loop_expected(x, skip, 256), rtol=1e-6, atol=1e-6)
    runtime_lib.Module(src, "branch_in_loop_kernel", NVRTC_OPTIONS)


OUT = np.zeros(8, dtype=np.float32)


@triton.jit
def block_condition_kernel(out, n):
    lanes = tl.arange(0, 8)
    if lanes < n:
        tl.store(out + lanes, 1.0)


@triton.jit
def one_sided_name_kernel(out, n):
    if n < 3:
        value = 1.0
    tl.store(out, value)


@triton.jit
def pointer_under_condition_kernel(out, other, n):
    target = out
    if n < 3:
        target = other
    tl.store(target, 1.0)


@triton.jit
def return_in_loop_kernel(out, n):
    for i in range(0, n):
        if i < 2:
            return
    tl.store(out, 1.0)


@triton.jit
def return_value_kernel(out, n):
    if n < 3:
        return 1
    tl.store(out, 1.0)


@triton.jit
def numeric_condition_kernel(out, n):
    if n:
        tl.store(out, 1.0)


@pytest.mark.parametrize("kernel,args,message", [
    (block_condition_kernel, (OUT, 3), "scalar boolean"),
    (one_sided_name_kernel, (OUT, 3), "only one path"),
    (pointer_under_condition_kernel, (OUT, OUT, 3), "pointer 'target'"),
    (return_in_loop_kernel, (OUT, 3), "return inside a runtime loop"),
    (return_value_kernel, (OUT, 3), "return statements are not supported"),
    (numeric_condition_kernel, (OUT, 3), "scalar boolean"),
])
def test_what_stays_rejected(kernel, args, message):
    with pytest.raises(ASTFrontendError, match=message):
        kernel[(1,)](*args)


@triton.jit
def same_on_both_paths_kernel(out, n, FLAG: tl.constexpr):
    scale = 2.0
    if n < 3:
        scale = 2.0
        width = FLAG
    else:
        width = FLAG
    tl.store(out + width, scale)


def test_names_bound_to_equal_constants_stay_constants():
    _, ssa_ops, _ = same_on_both_paths_kernel[(1,)](OUT, 5, FLAG=4)
    assert [op.opcode for op in ssa_ops] == ["addptr", "store"]       # no select was needed


def collatz_expected(programs, limit):
    out = np.zeros(programs, np.float32)
    for pid in range(programs):
        value, steps = pid + 1, 0
        while value > 1 and steps < limit:
            value = value * 3 + 1 if value % 2 else value // 2
            steps += 1
        out[pid] = steps
    return out


def while_chunks_expected(x, budget, block):
    rows, cols = x.shape
    out = np.zeros((rows, 2), np.float32)
    for r in range(rows):
        acc, start, spent = np.zeros(block, np.float32), 0, np.float32(0.0)
        while start < cols and spent < budget:
            piece = np.zeros(block, np.float32)
            chunk = x[r, start:start + block]
            piece[:len(chunk)] = chunk
            acc += piece
            spent = np.float32(spent + ssa_interp.tree_sum(np.abs(piece)))
            start += block
        out[r] = ssa_interp.tree_sum(acc), start
    return out


def test_while_loops_are_counted_loops_that_leave_on_a_false_condition(runtime_lib):
    out = np.zeros(40, np.float32)
    _, ssa_ops, src = corpus.collatz_kernel[(40,)](out, 1000)
    text = SSAPrinter().print_ops(ssa_ops)
    assert "in range(0, 2147483647, 1)" in text and "break_unless" in text
    ssa_interp.run(text, {"out": out, "limit": 1000}, (40,))
    np.testing.assert_array_equal(out, collatz_expected(40, 1000))
    assert out[26] == 111                                    # 27 takes 111 steps
    out[:] = 0
    ssa_interp.run(text, {"out": out, "limit": 5}, (40,))
    np.testing.assert_array_equal(out, collatz_expected(40, 5))
    assert "break;" in src
    runtime_lib.Module(src, "collatz_kernel", NVRTC_OPTIONS)


@pytest.mark.parametrize("budget", [0.0, 300.0, 1e9])
def test_while_condition_fed_by_a_reduction_in_the_body(budget, runtime_lib):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((4, 1500)).astype(np.float32)
    out = np.zeros((4, 2), np.float32)
    _, ssa_ops, src = corpus.while_chunks_kernel[(4,)](x, out, 1500, budget, BLOCK=256)
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {"x": x, "out": out, "n_cols": 1500, "budget": budget}, (4,))
    np.testing.assert_allclose(out, while_chunks_expected(x, budget, 256), rtol=1e-6, atol=1e-6)
    runtime_lib.Module(src, "while_chunks_kernel", NVRTC_OPTIONS)


@triton.jit
def while_true_kernel(out, n):
    while True:
        tl.store(out, 1.0)


@triton.jit
def while_else_kernel(out, n):
    while n < 3:
        n = n + 1
    else:
        tl.store(out, 1.0)


@triton.jit
def while_block_condition_kernel(out, n):
    lanes = tl.arange(0, 8)
    while lanes < n:
        n = n - 1


@triton.jit
def while_in_untaken_branch_kernel(out, n):
    """The loop below never ends by itself; under a false branch condition it must."""
    count = 0
    if n < 0:
        while count < 1000000:
            count = count + 0
    tl.store(out, count)


@pytest.mark.parametrize("kernel,message", [
    (while_true_kernel, "must depend on run-time values"),
    (while_else_kernel, "while/else"),
    (while_block_condition_kernel, "scalar boolean"),
])
def test_while_forms_that_stay_rejected(kernel, message):
    with pytest.raises(ASTFrontendError, match=message):
        kernel[(1,)](OUT, 3)


def test_a_loop_in_a_branch_that_is_not_taken_ends_at_once():
    out = np.full(1, 7.0, np.float32)
    _, ssa_ops, _ = while_in_untaken_branch_kernel[(1,)](out, 5)
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {"out": out, "n": 5}, (1,))
    assert out[0] == 0


def test_break_unless_is_verified():
    from mytriton_b200.nodes import Param
    from mytriton_b200.ssa import SSAOp
    from mytriton_b200.ssa_verification import CompileError, SSAVerifier
    from mytriton_b200.types import I32

    with pytest.raises(CompileError, match="outside a loop body"):
        SSAVerifier(None).verify([SSAOp("break_unless", (Param("n", I32),))])


@triton.jit
def remainder_kernel(out, n, DIVISOR: tl.constexpr):
    lanes = tl.arange(0, 16)
    values = lanes - n
    tl.store(out + lanes, values % DIVISOR)
    tl.store(out + 16 + lanes, values // DIVISOR)
    tl.store(out + 32 + lanes, (values % n) + (7 % 3) + (7 // 2))


def test_remainder_and_floor_division_follow_c(runtime_lib):
    """% and // on i32 are C's: the remainder takes the dividend's sign, division truncates."""
    out = np.zeros(48, np.float32)
    _, ssa_ops, src = remainder_kernel[(1,)](out, 5, DIVISOR=3)
    opcodes = [op.opcode for op in ssa_ops]
    assert "rem" in opcodes and "div" in opcodes
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {"out": out, "n": 5}, (1,))
    values = np.arange(16) - 5
    assert np.array_equal(out[:16], np.fmod(values, 3))
    assert np.array_equal(out[16:32], np.trunc(values / 3))
    assert np.array_equal(out[32:], np.fmod(values, 5) + 1 + 3)
    assert " % " in src
    runtime_lib.Module(src, "remainder_kernel", NVRTC_OPTIONS)
    with pytest.raises(TypeError, match="expects i32"):
        float_remainder_kernel[(1,)](out, 2.5)


@triton.jit
def float_remainder_kernel(out, x):
    tl.store(out, x % 2)


@triton.jit
def leaky_helper(x, slope):
    return tl.where(x < 0.0, x * slope, x)


@triton.jit
def store_scaled_helper(ptr, value, mask, SCALE: tl.constexpr):
    tl.store(ptr, value * SCALE, mask=mask)


@triton.jit
def chunk_sum_helper(x, row, n_cols, BLOCK: tl.constexpr):
    lanes = tl.arange(0, BLOCK)
    acc = tl.zeros((BLOCK,), tl.float32)
    for start in range(0, n_cols, BLOCK):
        cols = start + lanes
        acc = acc + tl.load(x + row * n_cols + cols, mask=cols < n_cols, other=0.0)
    return tl.sum(acc)


@triton.jit
def calls_helpers_kernel(x, out, sums, n_cols, slope, BLOCK: tl.constexpr):
    row = tl.program_id(0)
    offs = tl.arange(0, BLOCK)
    mask = offs < n_cols
    v = leaky_helper(tl.load(x + row * n_cols + offs, mask=mask, other=0.0), slope=slope)
    store_scaled_helper(out + row * n_cols + offs, v, mask, SCALE=3.0)
    tl.store(sums + row, chunk_sum_helper(x, row, n_cols, BLOCK=BLOCK))


@triton.jit
def early_return_helper(x, n):
    if n < 3:
        return x
    return x + 1.0


@triton.jit
def calls_bad_helper_kernel(out, n):
    tl.store(out, early_return_helper(2.0, n))


def test_jit_functions_called_from_a_kernel_are_traced_in_place(runtime_lib):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 100)).astype(np.float32)
    out, sums = np.zeros_like(x), np.zeros(3, np.float32)
    _, ssa_ops, src = calls_helpers_kernel[(3,)](x, out, sums, 100, 0.1, BLOCK=128)
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops),
                   {"x": x, "out": out, "sums": sums, "n_cols": 100, "slope": 0.1}, (3,))
    np.testing.assert_array_equal(out, np.where(x < 0, x * np.float32(0.1), x) * np.float32(3.0))
    np.testing.assert_allclose(sums, x.sum(axis=1), rtol=1e-5, atol=1e-5)
    runtime_lib.Module(src, "calls_helpers_kernel", NVRTC_OPTIONS)
    with pytest.raises(ASTFrontendError, match="may not return from inside a run-time if"):
        calls_bad_helper_kernel[(1,)](OUT, 5)
    with pytest.raises(ASTFrontendError, match="leaky_helper"):
        bad_arity_kernel[(1,)](OUT, 5)


@triton.jit
def bad_arity_kernel(out, n):
    tl.store(out, leaky_helper(2.0))


@triton.jit
def math_functions_kernel(x, out, n, BLOCK: tl.constexpr):
    """The f32 functions beyond exp, abs on both element types, sigmoid and cdiv."""
    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
    mask = offs < n
    v = tl.load(x + offs, mask=mask, other=1.0)
    positive = tl.abs(v) + 0.5
    y = tl.sqrt(positive) + tl.rsqrt(positive) + tl.log(positive) + tl.log2(positive) + tl.exp2(v * 0.25)
    y = y + tl.sin(v) + tl.cos(v) + tl.tanh(v) + tl.sigmoid(v) + tl.abs(offs - 7) + tl.cdiv(BLOCK, 3)
    tl.store(out + offs, y, mask=mask)


def math_functions_expected(x, block):
    positive = np.abs(x) + np.float32(0.5)
    y = np.sqrt(positive) + 1 / np.sqrt(positive) + np.log(positive) + np.log2(positive) + np.exp2(x * np.float32(0.25))
    y = y + np.sin(x) + np.cos(x) + np.tanh(x) + 1 / (1 + np.exp(-x)) + np.abs(np.arange(len(x)) - 7) + -(-block // 3)
    return y.astype(np.float32)


def test_math_functions(runtime_lib):
    rng = np.random.default_rng(9)
    x = (rng.standard_normal(300) * 2).astype(np.float32)
    out = np.zeros_like(x)
    _, ssa_ops, src = math_functions_kernel[(3,)](x, out, 300, BLOCK=128)
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {"x": x, "out": out, "n": 300}, (3,))
    np.testing.assert_allclose(out, math_functions_expected(x, 128), rtol=1e-5, atol=1e-5)
    for function in ("sqrtf", "rsqrtf", "logf", "log2f", "exp2f", "sinf", "cosf", "tanhf", "fabsf"):
        assert function + "(" in src
    runtime_lib.Module(src, "math_functions_kernel", NVRTC_OPTIONS)
    with pytest.raises(TypeError, match="sqrt requires f32"):
        integer_sqrt_kernel[(1,)](OUT, 3)


@triton.jit
def integer_sqrt_kernel(out, n):
    tl.store(out, tl.sqrt(n))


def test_layer_norm_kernel_in_the_oracle(runtime_lib):
    rng = np.random.default_rng(3)
    x = (rng.standard_normal((6, 100)) * 3 + 1).astype(np.float32)
    weight, bias = rng.standard_normal(100).astype(np.float32), rng.standard_normal(100).astype(np.float32)
    out = np.zeros_like(x)
    _, ssa_ops, src = corpus.layer_norm_kernel[(6,)](x, weight, bias, out, 100, 1e-5, BLOCK=128)
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops),
                   {"x": x, "weight": weight, "bias": bias, "out": out, "n_cols": 100, "eps": 1e-5}, (6,))
    x64 = x.astype(np.float64)
    mean = x64.mean(axis=1, keepdims=True)
    want = (x64 - mean) / np.sqrt(((x64 - mean) ** 2).mean(axis=1, keepdims=True) + 1e-5) * weight + bias
    np.testing.assert_allclose(out, want, rtol=1e-4, atol=1e-5)
    assert "rsqrtf(" in src
    runtime_lib.Module(src, "layer_norm_kernel", NVRTC_OPTIONS)


@triton.jit
def histogram_kernel(x, bins, total, n, BLOCK: tl.constexpr):
    """tl.atomic_add: three buckets (negative, [0, 1), the rest) and a grand total, both
    accumulated across programs."""
    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
    mask = offs < n
    v = tl.load(x + offs, mask=mask, other=0.0)
    bucket = tl.where(v < 0.0, offs * 0, offs * 0 + 1) + tl.where(v < 1.0, offs * 0, offs * 0 + 1)
    tl.atomic_add(bins + bucket, 1.0, mask=mask)
    tl.atomic_add(total, tl.sum(tl.where(mask, v, 0.0)))


def test_atomic_add(runtime_lib):
    x = np.random.default_rng(0).standard_normal(1000).astype(np.float32)
    bins, total = np.zeros(3, np.float32), np.zeros(1, np.float32)
    _, ssa_ops, src = histogram_kernel[(4,)](x, bins, total, 1000, BLOCK=256)
    assert [op.opcode for op in ssa_ops].count("atomic_add") == 2
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {"x": x, "bins": bins, "total": total, "n": 1000}, (4,))
    assert bins.tolist() == [(x < 0).sum(), ((x >= 0) & (x < 1)).sum(), (x >= 1).sum()]
    np.testing.assert_allclose(total[0], x.sum(), rtol=1e-5)
    assert src.count("atomicAdd(&") == 2
    runtime_lib.Module(src, "histogram_kernel", NVRTC_OPTIONS)
    from mytriton_b200.optim import ConstantFoldPass, CSEPass, DCEPass, PassManager
    from mytriton_b200.ssa_verification import SSAVerifier

    kept = PassManager([ConstantFoldPass(), CSEPass(), DCEPass()], SSAVerifier(None)).run(list(ssa_ops))
    assert [op.opcode for op in kept].count("atomic_add") == 2          # side effects survive DCE


def tile_softmax_expected(x):
    peak = x.max(axis=1, keepdims=True)
    e = np.exp(x - peak)
    total = e.sum(axis=1, keepdims=True)
    return (e / total).astype(np.float32), np.concatenate([total, peak], axis=1).astype(np.float32)


@pytest.mark.parametrize("tile,options", [((8, 64), {}), ((16, 128), {"num_warps": 4}), ((4, 512), {}),
                                          ((32, 16), {"num_warps": 1}), ((2, 8), {})])
def test_reductions_along_the_last_axis_of_a_tile(tile, options, runtime_lib):
    """Row reductions of a rank-2 block, used broadcast over the tile and as vectors; the
    tiles cover the in-warp shuffle geometry, rows that span warps, and tiny CTAs."""
    bm, bn = tile
    rng = np.random.default_rng(bm * bn)
    n_rows, n_cols = 3 * bm - 1, bn - 3
    x = (rng.standard_normal((n_rows, n_cols)) * 3).astype(np.float32)
    out, stats = np.zeros_like(x), np.zeros((n_rows, 2), np.float32)
    grid = (-(-n_rows // bm),)
    _, ssa_ops, src = corpus.tile_softmax_kernel[grid](x, out, stats, n_rows, n_cols, BM=bm, BN=bn, **options)
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops),
                   {"x": x, "out": out, "stats": stats, "n_rows": n_rows, "n_cols": n_cols}, grid)
    want_out, want_stats = tile_softmax_expected(x)
    np.testing.assert_allclose(out, want_out, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(stats, want_stats, rtol=1e-5, atol=1e-6)
    runtime_lib.Module(src, "tile_softmax_kernel", NVRTC_OPTIONS)


@triton.jit
def column_sum_kernel(x, out, BM: tl.constexpr, BN: tl.constexpr):
    rows = tl.arange(0, BM)
    cols = tl.arange(0, BN)
    tl.store(out + cols, tl.sum(tl.load(x + rows[:, None] * BN + cols[None, :]), axis=0))


@pytest.mark.parametrize("tile", [(8, 16), (32, 64), (6, 10)])
def test_reduction_along_the_first_axis(tile, runtime_lib):
    bm, bn = tile
    x = np.random.default_rng(bm).standard_normal((bm, bn)).astype(np.float32)
    out = np.zeros(bn, np.float32)
    _, ssa_ops, src = column_sum_kernel[(1,)](x, out, BM=bm, BN=bn)
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {"x": x, "out": out}, (1,))
    np.testing.assert_allclose(out, x.sum(axis=0), rtol=1e-5, atol=1e-5)
    runtime_lib.Module(src, "column_sum_kernel", NVRTC_OPTIONS)


def attention_expected(q, k, v, scale):
    scores = (q.astype(np.float64) @ k.astype(np.float64).T) * scale
    weights = np.exp(scores - scores.max(axis=1, keepdims=True))
    return ((weights / weights.sum(axis=1, keepdims=True)) @ v.astype(np.float64)).astype(np.float32)


def test_streaming_attention_kernel(runtime_lib):
    rng = np.random.default_rng(12)
    seq, d = 45, 16
    q, k, v = (rng.standard_normal((seq, d)).astype(np.float32) for _ in range(3))
    out = np.zeros_like(q)
    _, ssa_ops, src = corpus.attention_kernel[(3,)](q, k, v, out, seq, 0.25, BM=16, BN=16, D=16)
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops),
                   {"q": q, "k": k, "v": v, "out": out, "seq": seq, "scale": 0.25}, (3,))
    np.testing.assert_allclose(out, attention_expected(q, k, v, 0.25), rtol=1e-5, atol=1e-5)
    runtime_lib.Module(src, "attention_kernel", NVRTC_OPTIONS)


# ---------------------------------------------------------------- break / continue


def scan_until_expected(x, limit, block):
    rows = []
    for r in x:
        total, visited, stopped = np.float32(0.0), 0, -1
        for start in range(0, len(r), block):
            visited += 1
            if r[start] < 0:
                continue
            chunk = r[start:start + block].sum(dtype=np.float32)       # small integers: exact in any order
            if chunk > limit:
                stopped = start
                break
            total += chunk
        rows.append((total, visited, stopped))
    return np.array(rows, np.float32)


def first_negative_expected(x):
    rows = []
    for r in x:
        negative = np.flatnonzero(r < 0)
        index = int(negative[0]) if len(negative) else len(r)
        rows.append((r[:index].sum(dtype=np.float32), index))
    return np.array(rows, np.float32)


def nested_break_expected(x, limit, block):
    counted, grand = 0, np.float32(0.0)
    for r in x:
        total = np.float32(0.0)
        for start in range(0, len(r), block):
            chunk = r[start:start + block].sum(dtype=np.float32)
            if chunk < 0:
                break
            total += chunk
        if total > limit:
            continue
        counted += 1
        grand += total
    firsts = np.float32(0.0)
    for value in x.reshape(-1)[:4]:
        if value < 0:
            break
        firsts += value
    return np.array([grand, counted, firsts], np.float32)


@pytest.mark.parametrize("limit", [-1000.0, 150.0, 230.0, 1e9])
def test_break_and_continue_in_a_runtime_loop(limit, runtime_lib):
    """`continue` skips the rest of the body under a flag, `break` sets a flag that is carried
    through the loop and tested (`break_unless`) where the next iteration starts."""
    rng = np.random.default_rng(11)
    x = rng.integers(-2, 6, (7, 1000)).astype(np.float32)
    out = np.zeros((7, 3), np.float32)
    _, ssa_ops, src = corpus.scan_until_kernel[(7,)](x, out, 1000, limit, BLOCK=128)
    text = SSAPrinter().print_ops(ssa_ops)
    header = next(line for line in text.splitlines() if " for " in line)
    assert "break_unless" in text and "= False" in header and "bool" in header     # the flag is carried
    ssa_interp.run(text, {"x": x, "out": out, "n_cols": 1000, "limit": limit}, (7,))
    np.testing.assert_array_equal(out, scan_until_expected(x, limit, 128))
    runtime_lib.Module(src, "scan_until_kernel", NVRTC_OPTIONS)


def test_while_true_is_left_by_break(runtime_lib):
    rng = np.random.default_rng(12)
    x = rng.integers(-1, 9, (6, 40)).astype(np.float32)
    x[2] = np.abs(x[2])                                          # no negative value: runs to the end
    x[4, 0] = -1.0                                               # leaves at once
    out = np.zeros((6, 2), np.float32)
    _, ssa_ops, src = corpus.first_negative_kernel[(6,)](x, out, 40)
    text = SSAPrinter().print_ops(ssa_ops)
    assert text.count("break_unless") == 1                       # only the break's flag is tested
    ssa_interp.run(text, {"x": x, "out": out, "n": 40}, (6,))
    np.testing.assert_array_equal(out, first_negative_expected(x))
    runtime_lib.Module(src, "first_negative_kernel", NVRTC_OPTIONS)


@pytest.mark.parametrize("limit", [0.0, 400.0, 1e9])
def test_an_inner_break_leaves_only_the_inner_loop(limit, runtime_lib):
    rng = np.random.default_rng(13)
    x = rng.integers(-3, 7, (9, 700)).astype(np.float32)
    x[0, :4] = (2.0, 3.0, -1.0, 5.0)                             # the unrolled loop breaks at its third step
    out = np.zeros(3, np.float32)
    _, ssa_ops, src = corpus.nested_break_kernel[(1,)](x, out, 9, 700, limit, BLOCK=64)
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops),
                   {"x": x, "out": out, "n_rows": 9, "n_cols": 700, "limit": limit}, (1,))
    np.testing.assert_array_equal(out, nested_break_expected(x, limit, 64))
    assert out[2] == 5.0
    runtime_lib.Module(src, "nested_break_kernel", NVRTC_OPTIONS)


@triton.jit
def compile_time_break_kernel(out, n, STOP: tl.constexpr):
    total = 0.0
    for k in range(8):
        if k == STOP:
            break
        if k == 1:
            continue
        total += 1.0
    tl.store(out, total)


def test_break_on_a_compile_time_condition_unrolls_to_nothing_more():
    """In an unrolled loop with compile-time conditions the flags are Python values: no select, no
    flag arithmetic reaches the IR."""
    out = np.zeros(1, np.float32)
    _, ssa_ops, _ = compile_time_break_kernel[(1,)](out, 0, STOP=5)
    text = SSAPrinter().print_ops(ssa_ops)
    assert "select" not in text and "not" not in text
    ssa_interp.run(text, {"out": out, "n": 0}, (1,))
    assert out[0] == 4.0                                         # k = 0, 2, 3, 4


def _random_jump_body(rng, depth, loop_depth, indent):
    """Statements over the integers acc, cnt and the loop indices: assignments, if / else, guarded
    `break` / `continue`, and (once) an inner loop."""
    pad = "    " * indent
    lines = []
    for _ in range(int(rng.integers(1, 4))):
        kind = rng.choice(["assign", "assign", "if", "jump", "loop"] if depth < 3 else ["assign", "jump"])
        if kind == "assign":
            target = rng.choice(["acc", "cnt"])
            addend = rng.choice(["i", "a", "1", "2", "j"] if loop_depth > 1 else ["i", "a", "1", "2"])
            lines.append(f"{pad}{target} = {target} + {addend}")
        elif kind == "if":
            test = rng.choice(["i < a", "acc > b", "cnt < 3", "i > 2", "not acc < a", "(i < b) & (cnt < 5)"])
            lines.append(f"{pad}if {test}:")
            lines += _random_jump_body(rng, depth + 1, loop_depth, indent + 1)
            if rng.random() < 0.5:
                lines.append(f"{pad}else:")
                lines += _random_jump_body(rng, depth + 1, loop_depth, indent + 1)
        elif kind == "jump":
            lines.append(f"{pad}if {rng.choice(['i > a', 'acc > b', 'cnt > 4', 'i < 1'])}:")
            if rng.random() < 0.4:
                lines.append(f"{pad}    cnt = cnt + 1")
            lines.append(f"{pad}    {rng.choice(['break', 'continue'])}")
        elif loop_depth == 1:
            lines.append(f"{pad}for j in range(0, a):")
            lines += [line.replace(" i ", " j ").replace("i <", "j <").replace("i >", "j >")
                      for line in _random_jump_body(rng, depth + 1, 2, indent + 1)]
        else:
            lines.append(f"{pad}acc = acc + 1")
    return lines


def jump_case(seed, tmp_path):
    """(kernel, the same statements as a Python function, source) for one seed."""
    import importlib.util

    rng = np.random.default_rng(900 + seed)
    body = _random_jump_body(rng, 0, 1, 2)
    if rng.random() < 0.3:          # the index moves first, so that `continue` cannot loop forever
        loop = ["    i = 0", "    while i < n:", "        i = i + 1"] + body
    else:
        loop = ["    for i in range(0, n):"] + body
    statements = ["    acc = 0", "    cnt = 0", "    j = 0"] + loop
    source = "\n".join(["import mytriton_b200 as triton", "import mytriton_b200.language as tl", "", "",
                        "@triton.jit", "def jumps_kernel(out, n, a, b):"] + statements
                       + ["    tl.store(out, acc * 1.0)", "    tl.store(out + 1, cnt * 1.0)"]) + "\n"
    path = tmp_path / f"jumps_{seed}.py"
    path.write_text(source)
    spec = importlib.util.spec_from_file_location(path.stem, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    plain: dict = {}
    exec("\n".join(["def reference(n, a, b):"] + statements + ["    return acc, cnt"]).replace(" & ", " and "), plain)
    return module.jumps_kernel, plain["reference"], source


JUMP_ARGUMENTS = ((0, 1, 5), (5, 2, 7), (9, 3, 20), (12, 0, 3))


@pytest.mark.parametrize("seed", range(40))
def test_random_loops_with_jumps_mean_what_python_means(seed, tmp_path):
    """Random scalar loops (for and while, nested, with if / else, break and continue): the lowered
    kernel run by the SSA interpreter gives what the same statements give as plain Python."""
    kernel, reference, source = jump_case(seed, tmp_path)
    for n, a, b in JUMP_ARGUMENTS:
        out = np.zeros(2, np.float32)
        _, ssa_ops, _ = kernel[(1,)](out, n, a, b)
        ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {"out": out, "n": n, "a": a, "b": b}, (1,))
        assert tuple(out) == reference(n, a, b), source


@triton.jit
def equality_kernel(x, out, n, k, BLOCK: tl.constexpr):
    pid = tl.program_id(0)
    offs = pid * BLOCK + tl.arange(0, BLOCK)
    v = tl.load(x + offs, mask=offs < n, other=0.0)
    if pid == k:
        v = v * 2.0
    if pid != 0:
        v = v + 1.0
    v = tl.where(offs % 3 == 0, v, -v)
    tl.store(out + offs, v, mask=offs < n)


@triton.jit
def float_equality_kernel(x, out):
    v = tl.load(x)
    if v == 1.0:
        tl.store(out, v)


def equality_expected(x, k, block):
    want = x.copy()
    want[k * block:(k + 1) * block] *= 2
    want[block:] += 1
    return np.where(np.arange(len(x)) % 3 == 0, want, -want)


def test_integer_equality_on_runtime_values(runtime_lib):
    """`==` and `!=` between integers, scalars or blocks, are "neither is smaller" (and its
    negation); floating-point operands are refused, because that would call NaN equal to itself."""
    x = np.arange(40, dtype=np.float32)
    out = np.zeros(40, np.float32)
    _, ssa_ops, src = equality_kernel[(5,)](x, out, 40, 2, BLOCK=8)
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {"x": x, "out": out, "n": 40, "k": 2}, (5,))
    np.testing.assert_array_equal(out, equality_expected(x, 2, 8))
    runtime_lib.Module(src, "equality_kernel", NVRTC_OPTIONS)
    with pytest.raises(ASTFrontendError, match="integers only"):
        float_equality_kernel[(1,)](x, out)


@pytest.mark.parametrize("programs", [1, 3, 40])
def test_num_programs_lets_a_fixed_grid_stride_over_the_work(programs, runtime_lib):
    x = np.arange(1000, dtype=np.float32)
    out = np.zeros_like(x)
    _, ssa_ops, src = corpus.strided_scale_kernel[(programs,)](x, out, 1000, 3.0, BLOCK=64)
    text = SSAPrinter().print_ops(ssa_ops)
    assert "num_programs {axis=0} : i32" in text
    ssa_interp.run(text, {"x": x, "out": out, "n": 1000, "factor": 3.0}, (programs,))
    np.testing.assert_array_equal(out, 3 * x)
    assert "gridDim.x" in src
    runtime_lib.Module(src, "strided_scale_kernel", NVRTC_OPTIONS)


@triton.jit
def rounding_kernel(x, out16, outb, n, BLOCK: tl.constexpr):
    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
    v = tl.load(x + offs, mask=offs < n, other=0.0)
    tl.store(out16 + offs, (v * 3.0).to(tl.float16) + offs.to(tl.float32), mask=offs < n)
    tl.store(outb + offs, v.to(tl.bfloat16).to(tl.float32), mask=offs < n)


def rounding_expected(x):
    import ml_dtypes

    half = (x * np.float32(3.0)).astype(np.float16).astype(np.float32) + np.arange(len(x), dtype=np.float32)
    return half, x.astype(ml_dtypes.bfloat16).astype(np.float32)


def test_to_rounds_to_the_named_precision(runtime_lib):
    """`x.to(tl.float16)` / `x.to(tl.bfloat16)` round to nearest even and stay fp32 in registers;
    `.to(tl.float32)` turns integers into floats; float -> int is refused."""
    x = (np.random.default_rng(3).standard_normal(100) * 50).astype(np.float32)
    out16, outb = np.zeros(100, np.float32), np.zeros(100, np.float32)
    _, ssa_ops, src = rounding_kernel[(2,)](x, out16, outb, 100, BLOCK=64)
    text = SSAPrinter().print_ops(ssa_ops)
    assert "round_f16" in text and "round_bf16" in text
    ssa_interp.run(text, {"x": x, "out16": out16, "outb": outb, "n": 100}, (2,))
    want16, wantb = rounding_expected(x)
    np.testing.assert_array_equal(out16, want16)
    np.testing.assert_array_equal(outb, wantb)
    runtime_lib.Module(src, "rounding_kernel", NVRTC_OPTIONS)
    with pytest.raises(TypeError, match="to int32"):
        (tl.program_id(0) * 1.5).to(tl.int32)


@triton.jit
def transpose_kernel(x, out, M, N, BM: tl.constexpr, BN: tl.constexpr):
    """out[N, M] = 2 * x[M, N].T, tile by tile."""
    rows = tl.program_id(0) * BM + tl.arange(0, BM)
    cols = tl.program_id(1) * BN + tl.arange(0, BN)
    tile = tl.load(x + rows[:, None] * N + cols[None, :], mask=(rows[:, None] < M) & (cols[None, :] < N), other=0.0)
    tl.store(out + cols[:, None] * M + rows[None, :], tl.trans(tile) * 2.0,
             mask=(cols[:, None] < N) & (rows[None, :] < M))


@triton.jit
def scores_kernel(q, k, s, n, D: tl.constexpr, B: tl.constexpr):
    """s = q @ k.T, tile by tile: the second operand of the dot is a transposed tile."""
    i = tl.program_id(0) * B + tl.arange(0, B)
    j = tl.program_id(1) * B + tl.arange(0, B)
    d = tl.arange(0, D)
    q_tile = tl.load(q + i[:, None] * D + d[None, :], mask=i[:, None] < n, other=0.0)
    k_tile = tl.load(k + j[:, None] * D + d[None, :], mask=j[:, None] < n, other=0.0)
    tl.store(s + i[:, None] * n + j[None, :], tl.dot(q_tile, tl.trans(k_tile)),
             mask=(i[:, None] < n) & (j[None, :] < n))


def test_trans_exchanges_the_coordinates_of_what_produces_the_block(runtime_lib):
    rng = np.random.default_rng(14)
    x = rng.standard_normal((50, 70)).astype(np.float32)
    out = np.zeros((70, 50), np.float32)
    _, ssa_ops, src = transpose_kernel[(4, 5)](x, out, 50, 70, BM=16, BN=16)
    text = SSAPrinter().print_ops(ssa_ops)
    assert "trans %" in text and "block<16x16 x f32>" in text
    ssa_interp.run(text, {"x": x, "out": out, "M": 50, "N": 70}, (4, 5))
    np.testing.assert_array_equal(out, 2 * x.T)
    runtime_lib.Module(src, "transpose_kernel", NVRTC_OPTIONS)
    q, k = rng.standard_normal((40, 16)).astype(np.float32), rng.standard_normal((40, 16)).astype(np.float32)
    s = np.zeros((40, 40), np.float32)
    _, ssa_ops, src = scores_kernel[(3, 3)](q, k, s, 40, D=16, B=16)
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {"q": q, "k": k, "s": s, "n": 40}, (3, 3))
    np.testing.assert_allclose(s, q @ k.T, atol=1e-5)
    runtime_lib.Module(src, "scores_kernel", NVRTC_OPTIONS)
    from mytriton_b200.type_inference import TypeInference

    with pytest.raises(TypeError, match="rank-2"):
        TypeInference().infer(tl.trans(tl.arange(0, 8)).expr)
