"""Run-time if / else / not / return on the GPU against the closed forms of
tests/test_control_flow.py (elementwise part bit-exact; block sums to 1e-5 relative to the
sum of magnitudes, because the device adds in a different order)."""

import numpy as np
import pytest

from mytriton_b200 import kernels as corpus
from mytriton_b200 import device, runtime
from test_control_flow import branch_in_loop_expected, branchy_expected

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("block,options", [(256, {}), (1024, {"num_warps": 2}), (64, {"elems_per_thread": 2})])
@pytest.mark.parametrize("threshold", [0, 3, 100])
def test_branchy_kernel(block, options, threshold, gpu):
    rng = np.random.default_rng(block + threshold)
    n = 4 * block - 37
    x = rng.standard_normal(6 * block).astype(np.float32)
    dx, dout = device.to_device(x), device.to_device(np.full_like(x, 7.0))
    corpus.branchy_kernel[(6,)](dx, dout, n, threshold, BLOCK=block, **options)
    runtime.synchronize()
    got, want = dout.to_host(), branchy_expected(x, n, threshold, block)
    assert np.array_equal(got[n:], want[n:])                     # programs that returned wrote nothing
    scale = np.abs(x).reshape(6, block).sum(axis=1).repeat(block)
    assert np.all(np.abs(got - want) <= 1e-5 * np.maximum(scale, 1.0))
    exact = np.arange(len(x)) < min(threshold, 2) * block        # no block sum involved there
    assert np.array_equal(got[exact], want[exact])


@pytest.mark.parametrize("skip", [0, 1, 50])
@pytest.mark.parametrize("block", [128, 1024])
def test_branch_in_loop_kernel(skip, block, gpu):
    rng = np.random.default_rng(skip + block)
    x = rng.standard_normal((9, 3000)).astype(np.float32)
    dx, dout = device.to_device(x), device.to_device(np.zeros(9, np.float32))
    corpus.branch_in_loop_kernel[(9,)](dx, dout, 3000, skip, BLOCK=block)
    runtime.synchronize()
    want = branch_in_loop_expected(x, skip, block)
    scale = np.abs(x).sum(axis=1)
    assert np.all(np.abs(dout.to_host() - want) <= 1e-5 * scale)


def test_collatz_while_loop(gpu):
    from test_control_flow import collatz_expected

    for limit in (1000, 7):
        dout = device.to_device(np.zeros(300, np.float32))
        corpus.collatz_kernel[(300,)](dout, limit)
        runtime.synchronize()
        assert np.array_equal(dout.to_host(), collatz_expected(300, limit))


@pytest.mark.parametrize("block,options", [(256, {}), (2048, {"num_warps": 4}), (32, {})])
@pytest.mark.parametrize("budget", [0.0, 500.0, 1e9])
def test_while_with_a_reduction_in_its_condition(block, options, budget, gpu):
    """Every thread of the CTA must agree on when to leave: the reduced value is combined in
    one fixed order by all of them.  Budgets are placed away from any partial sum so that
    the different summation order of the device cannot move the exit."""
    from test_control_flow import while_chunks_expected

    rng = np.random.default_rng(block)
    x = rng.standard_normal((7, 5000)).astype(np.float32)
    want = while_chunks_expected(x, budget, block)
    dx, dout = device.to_device(x), device.to_device(np.zeros((7, 2), np.float32))
    corpus.while_chunks_kernel[(7,)](dx, dout, 5000, budget, BLOCK=block, **options)
    runtime.synchronize()
    got = dout.to_host()
    partial = np.cumsum(np.abs(x).reshape(7, -1)[:, : (5000 // block) * block].reshape(7, -1, block).sum(axis=2), axis=1) \
        if block <= 5000 else np.zeros((7, 1))
    if budget == 500.0 and np.min(np.abs(partial - budget)) < 1e-2:
        pytest.skip("a partial sum lands on the budget: the exit would depend on rounding")
    assert np.array_equal(got[:, 1], want[:, 1])                       # same number of chunks
    assert np.all(np.abs(got[:, 0] - want[:, 0]) <= 1e-5 * np.abs(x).sum(axis=1))


def test_remainder_and_floor_division(gpu):
    from test_control_flow import remainder_kernel

    dout = device.to_device(np.zeros(48, np.float32))
    remainder_kernel[(1,)](dout, 5, DIVISOR=3)
    runtime.synchronize()
    values = np.arange(16) - 5
    got = dout.to_host()
    assert np.array_equal(got[:16], np.fmod(values, 3))
    assert np.array_equal(got[16:32], np.trunc(values / 3))
    assert np.array_equal(got[32:], np.fmod(values, 5) + 1 + 3)


def test_math_functions(gpu):
    """sqrtf, rsqrtf, logf, ... against NumPy: 2e-6 relative to the magnitudes involved
    (the device's rsqrtf/tanhf/sinf are not correctly rounded)."""
    from test_control_flow import math_functions_expected, math_functions_kernel

    rng = np.random.default_rng(9)
    x = (rng.standard_normal(5000) * 2).astype(np.float32)
    dx, dout = device.to_device(x), device.to_device(np.zeros_like(x))
    math_functions_kernel[(5,)](dx, dout, 5000, BLOCK=1024)
    runtime.synchronize()
    want = math_functions_expected(x, 1024)
    assert np.all(np.abs(dout.to_host() - want) <= 2e-6 * np.maximum(np.abs(want), 5000.0))


@pytest.mark.parametrize("shape,block,options", [((37, 1000), 1024, {}), ((64, 4096), 4096, {"num_warps": 4}),
                                                 ((5, 17), 32, {})])
def test_layer_norm(shape, block, options, gpu):
    """A realistic row kernel on the new f32 functions: against an fp64 NumPy layer norm,
    1e-5 of the row's largest |y| (sums are reduced in a different order on the device)."""
    rows, cols = shape
    rng = np.random.default_rng(rows + cols)
    x = (rng.standard_normal((rows, cols)) * 3 + 1).astype(np.float32)
    weight = rng.standard_normal(cols).astype(np.float32)
    bias = rng.standard_normal(cols).astype(np.float32)
    dx, dw, db = device.to_device(x), device.to_device(weight), device.to_device(bias)
    dout = device.to_device(np.full_like(x, 7.0))
    corpus.layer_norm_kernel[(rows,)](dx, dw, db, dout, cols, 1e-5, BLOCK=block, **options)
    runtime.synchronize()
    x64 = x.astype(np.float64)
    mean = x64.mean(axis=1, keepdims=True)
    var = ((x64 - mean) ** 2).mean(axis=1, keepdims=True)
    want = (x64 - mean) / np.sqrt(var + 1e-5) * weight + bias
    got = dout.to_host()
    assert np.all(np.abs(got - want) <= 1e-5 * np.abs(want).max(axis=1, keepdims=True))


def test_atomic_add_across_programs(gpu):
    from test_control_flow import histogram_kernel

    x = np.random.default_rng(0).standard_normal(100_000).astype(np.float32)
    dx = device.to_device(x)
    bins, total = device.to_device(np.zeros(3, np.float32)), device.to_device(np.zeros(1, np.float32))
    histogram_kernel[(-(-len(x) // 1024),)](dx, bins, total, len(x), BLOCK=1024)
    runtime.synchronize()
    assert bins.to_host().tolist() == [(x < 0).sum(), ((x >= 0) & (x < 1)).sum(), (x >= 1).sum()]
    assert abs(total.to_host()[0] - x.astype(np.float64).sum()) <= 1e-5 * np.abs(x).sum()


@pytest.mark.parametrize("tile,options", [((8, 64), {}), ((16, 128), {"num_warps": 4}), ((4, 512), {}),
                                          ((32, 16), {"num_warps": 1}), ((2, 8), {}), ((64, 32), {"num_warps": 8})])
def test_reductions_along_the_last_axis_of_a_tile(tile, options, gpu):
    """Row maxima and sums of a [BM, BN] tile on the device: shuffle sub-groups where a row
    fits a warp, shared memory where it does not, and both uses of the result."""
    from test_control_flow import tile_softmax_expected

    bm, bn = tile
    rng = np.random.default_rng(bm * bn)
    n_rows, n_cols = 37 * bm - 1, bn - 3
    x = (rng.standard_normal((n_rows, n_cols)) * 3).astype(np.float32)
    dx = device.to_device(x)
    dout, dstats = device.to_device(np.zeros_like(x)), device.to_device(np.zeros((n_rows, 2), np.float32))
    corpus.tile_softmax_kernel[(-(-n_rows // bm),)](dx, dout, dstats, n_rows, n_cols, BM=bm, BN=bn, **options)
    runtime.synchronize()
    want_out, want_stats = tile_softmax_expected(x)
    np.testing.assert_allclose(dout.to_host(), want_out, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(dstats.to_host(), want_stats, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("seq,tile,options", [(45, (16, 16, 16), {}), (200, (32, 64, 32), {"num_warps": 4}),
                                              (130, (64, 32, 64), {"num_warps": 8}), (33, (8, 8, 8), {})])
def test_streaming_attention(seq, tile, options, gpu):
    """A flash-attention-style kernel written in the language: row reductions of score tiles,
    carried row vectors rescaling a carried accumulator, tl.dot on a computed operand.
    Against fp64 attention, 2e-5 of the output's scale."""
    from test_control_flow import attention_expected

    bm, bn, d = tile
    rng = np.random.default_rng(seq + d)
    q, k, v = (rng.standard_normal((seq, d)).astype(np.float32) for _ in range(3))
    dq, dk, dv = device.to_device(q), device.to_device(k), device.to_device(v)
    dout = device.to_device(np.full_like(q, 7.0))
    scale = float(1.0 / np.sqrt(d))
    corpus.attention_kernel[(-(-seq // bm),)](dq, dk, dv, dout, seq, scale, BM=bm, BN=bn, D=d, **options)
    runtime.synchronize()
    want = attention_expected(q, k, v, scale)
    assert np.all(np.abs(dout.to_host() - want) <= 2e-5 * max(1.0, float(np.abs(want).max())))


@pytest.mark.parametrize("tile", [(8, 16), (32, 64), (6, 10), (64, 128)])
def test_reduction_along_the_first_axis(tile, gpu):
    """Column sums of a tile (through shared memory) against NumPy."""
    from test_control_flow import column_sum_kernel

    bm, bn = tile
    x = np.random.default_rng(bm).standard_normal((bm, bn)).astype(np.float32)
    dx, dout = device.to_device(x), device.to_device(np.zeros(bn, np.float32))
    column_sum_kernel[(1,)](dx, dout, BM=bm, BN=bn)
    runtime.synchronize()
    np.testing.assert_allclose(dout.to_host(), x.astype(np.float64).sum(axis=0), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("block,options", [(128, {}), (1024, {"num_warps": 4}), (64, {"loop_passes": False})])
@pytest.mark.parametrize("limit", [-1000.0, 150.0, 1e9])
def test_break_and_continue(block, options, limit, gpu):
    """Small integers: every chunk sum is exact in any order, so the device must agree bit for bit
    with the closed form, including which chunk stops the scan."""
    from test_control_flow import scan_until_expected

    rng = np.random.default_rng(block)
    x = rng.integers(-2, 6, (33, 3000)).astype(np.float32)
    dx, dout = device.to_device(x), device.to_device(np.zeros((33, 3), np.float32))
    corpus.scan_until_kernel[(33,)](dx, dout, 3000, limit * block / 128, BLOCK=block, **options)
    runtime.synchronize()
    np.testing.assert_array_equal(dout.to_host(), scan_until_expected(x, limit * block / 128, block))


def test_while_true_with_break_and_nested_breaks(gpu):
    from test_control_flow import first_negative_expected, nested_break_expected

    rng = np.random.default_rng(21)
    x = rng.integers(-1, 9, (50, 64)).astype(np.float32)
    x[7] = np.abs(x[7])
    dx, dout = device.to_device(x), device.to_device(np.zeros((50, 2), np.float32))
    corpus.first_negative_kernel[(50,)](dx, dout, 64)
    runtime.synchronize()
    np.testing.assert_array_equal(dout.to_host(), first_negative_expected(x))

    y = rng.integers(-3, 7, (40, 1500)).astype(np.float32)
    y[0, :4] = (2.0, 3.0, -1.0, 5.0)
    dy = device.to_device(y)
    for limit in (0.0, 900.0, 1e9):
        dres = device.to_device(np.zeros(3, np.float32))
        corpus.nested_break_kernel[(1,)](dy, dres, 40, 1500, limit, BLOCK=256)
        runtime.synchronize()
        np.testing.assert_array_equal(dres.to_host(), nested_break_expected(y, limit, 256))


@pytest.mark.parametrize("seed", range(16))
def test_random_loops_with_jumps(seed, tmp_path, gpu):
    """The random scalar loops of the CPU test, compiled and run on the device."""
    from test_control_flow import JUMP_ARGUMENTS, jump_case

    kernel, reference, source = jump_case(seed, tmp_path)
    for n, a, b in JUMP_ARGUMENTS:
        dout = device.to_device(np.zeros(2, np.float32))
        kernel[(1,)](dout, n, a, b)
        runtime.synchronize()
        assert tuple(dout.to_host()) == reference(n, a, b), source


def test_integer_equality(gpu):
    from test_control_flow import equality_expected, equality_kernel

    x = np.arange(5000, dtype=np.float32)
    dx, dout = device.to_device(x), device.to_device(np.zeros_like(x))
    equality_kernel[(20,)](dx, dout, 5000, 7, BLOCK=256)
    runtime.synchronize()
    np.testing.assert_array_equal(dout.to_host(), equality_expected(x, 7, 256))


@pytest.mark.parametrize("programs", [1, 148, 1000])
def test_num_programs(programs, gpu):
    x = np.random.default_rng(programs).standard_normal(100_000).astype(np.float32)
    dx, dout = device.to_device(x), device.to_device(np.zeros_like(x))
    corpus.strided_scale_kernel[(programs,)](dx, dout, x.size, 3.0, BLOCK=512)
    runtime.synchronize()
    np.testing.assert_array_equal(dout.to_host(), np.float32(3.0) * x)


def test_to_rounds_on_the_device_as_numpy_does(gpu):
    from test_control_flow import rounding_expected, rounding_kernel

    x = (np.random.default_rng(4).standard_normal(10_000) * 50).astype(np.float32)
    x[:4] = (65504.0, 70000.0, 1e-8, -0.0)                     # fp16's largest value, overflow, underflow, -0
    dx = device.to_device(x)
    d16, db = device.to_device(np.zeros_like(x)), device.to_device(np.zeros_like(x))
    rounding_kernel[(-(-x.size // 256),)](dx, d16, db, x.size, BLOCK=256)
    runtime.synchronize()
    with np.errstate(over="ignore"):
        want16, wantb = rounding_expected(x)
    np.testing.assert_array_equal(d16.to_host(), want16)
    np.testing.assert_array_equal(db.to_host(), wantb)


@pytest.mark.parametrize("tile", [(16, 16), (32, 64), (8, 128)])
def test_trans(tile, gpu):
    from test_control_flow import scores_kernel, transpose_kernel

    bm, bn = tile
    rng = np.random.default_rng(bm + bn)
    x = rng.standard_normal((300, 500)).astype(np.float32)
    dx, dout = device.to_device(x), device.to_device(np.zeros((500, 300), np.float32))
    transpose_kernel[(-(-300 // bm), -(-500 // bn))](dx, dout, 300, 500, BM=bm, BN=bn)
    runtime.synchronize()
    np.testing.assert_array_equal(dout.to_host(), 2 * x.T)
    q, k = rng.standard_normal((100, 32)).astype(np.float32), rng.standard_normal((100, 32)).astype(np.float32)
    ds = device.to_device(np.zeros((100, 100), np.float32))
    scores_kernel[(7, 7)](device.to_device(q), device.to_device(k), ds, 100, D=32, B=16)
    runtime.synchronize()
    np.testing.assert_allclose(ds.to_host(), q.astype(np.float64) @ k.astype(np.float64).T, rtol=1e-5, atol=1e-4)
