"""Pins the CPU oracle against the known answers the reference's tests hold."""

import numpy as np

from oracle import numpy_oracle, ssa_interp


def run(golden, name, args, grid):
    ssa_interp.run(golden[name]["ssa"], args, grid)


def test_softmax_large_value_rows(golden):
    # tests/test_softmax_kernel.py:241-257
    x = np.array(
        [[1000.0, 1001.0, 999.0, 998.0], [-1000.0, -999.0, -1001.0, -1002.0],
         [1234.0, 1234.0, 1233.0, 1232.0]], dtype=np.float32)
    out = np.zeros((3, 8), dtype=np.float32)[:, :4].copy()
    run(golden, "softmax_8", {"x": x, "out": out, "n_cols": 4}, (3,))
    np.testing.assert_allclose(out, numpy_oracle.softmax(x), rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(out.sum(axis=1), 1.0, rtol=1e-6)
    e = np.exp(np.array([-1.0, 0.0, -2.0, -3.0]))
    np.testing.assert_allclose(out[0], e / e.sum(), rtol=1e-6)


def test_softmax_single_column_is_all_ones(golden):
    # tests/test_softmax_kernel.py:231-238
    x = np.random.default_rng(0).standard_normal((4, 1), dtype=np.float32)
    out = np.zeros_like(x)
    run(golden, "softmax_1", {"x": x, "out": out, "n_cols": 1}, (4,))
    assert np.array_equal(out, np.ones_like(x))


def test_extremum_table(golden):
    # tests/test_math_ops.py:270-291
    for lhs, rhs in [(np.nan, 2.0), (2.0, np.nan), (0.0, -0.0), (-0.0, 0.0), (3.0, 2.0), (2.0, 3.0)]:
        hi, lo = np.zeros(1, np.float32), np.zeros(1, np.float32)
        run(golden, "extremum", {"lhs": lhs, "rhs": rhs, "out_max": hi, "out_min": lo}, (1,))
        for got, want in ((hi[0], np.maximum(np.float32(lhs), np.float32(rhs))),
                          (lo[0], np.minimum(np.float32(lhs), np.float32(rhs)))):
            if np.isnan(want):
                assert np.isnan(got)
            else:
                assert got == want and np.signbit(got) == np.signbit(want)


def test_loop_closed_forms(golden):
    # tests/test_ast_runtime_loop.py:158-164 and :280-281
    n = 4
    out = np.zeros(1, np.float32)
    run(golden, "two_carried", {"out": out, "n": n}, (1,))
    first, second = 0, 1
    for k in range(n):
        first += k
        second += first
    assert out[0] == first + second
    out = np.zeros(1, np.float32)
    run(golden, "nested_loops", {"out": out, "n": n}, (1,))
    assert out[0] == n * n * (n - 1)
    out = np.zeros(3, np.float32)
    run(golden, "no_carried", {"out": out, "n": 3}, (1,))
    assert np.array_equal(out, [0.0, 1.0, 2.0])


def test_exact_integer_matmuls(golden):
    # tests/test_matmul_2d_kernel.py:175-190, tests/test_ast_runtime_loop.py:489-504
    M, N, K = 19, 23, 5
    a = np.arange(M * K, dtype=np.float32).reshape(M, K)
    b = np.arange(K * N, dtype=np.float32).reshape(K, N)
    for name, extra in (("matmul_runtime_k", {"K": K}), ("matmul_2d_k5", {})):
        c = np.zeros((M, N), np.float32)
        run(golden, name, {"a": a, "b": b, "c": c, "M": M, "N": N, **extra}, (3, 2))
        assert np.array_equal(c, a @ b)


def test_elementwise_against_numpy_expressions(golden):
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(1000, dtype=np.float32) * 2)
    x[:4] = [np.nan, 0.0, -0.0, -3.0]
    for name, args, expected in (
        ("relu_256", {}, numpy_oracle.relu(x)),
        ("leaky_relu_256", {"alpha": 0.01}, numpy_oracle.leaky_relu(x, 0.01)),
        ("sigmoid_256", {}, numpy_oracle.sigmoid(x)),
        ("copy_256", {}, numpy_oracle.copy(x)),
    ):
        out = np.full_like(x, 7.0)
        ordered = {"x": x.copy(), "out": out, "n": 1000, **args}
        run(golden, name, ordered, (4,))
        assert np.array_equal(out.view(np.uint32), expected.astype(np.float32).view(np.uint32)), name


def test_reductions_and_full(golden):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((127, 513), dtype=np.float32)
    for name, expected in (("row_sum_1024", numpy_oracle.row_sum(x)),
                           ("row_max_1024", numpy_oracle.row_max(x)),
                           ("row_min_1024", numpy_oracle.row_min(x))):
        out = np.zeros(127, np.float32)
        run(golden, name, {"x": x, "out": out, "n_cols": 513}, (127,))
        np.testing.assert_allclose(out, expected, rtol=1e-5, atol=1e-5)
    # tests/test_block_constructors.py:91-102
    for name, value in (("runtime_full_int", 3), ("runtime_full_float", 1.25)):
        out = np.zeros(5, np.float32)
        run(golden, name, {"out": out, "n": 5, "value": value}, (1,))
        assert np.array_equal(out, np.full(5, value, np.float32))


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.3895314e38], dtype=np.float32)
    r = numpy_oracle.round_to_bf16(x)
    assert r[0] == 1.0
    assert r[1] == 1.0            # exactly halfway between 1.0 and 1.0078125 -> even
    assert r[2] == np.float32(1.015625)   # halfway between 1.0078125 and 1.015625 -> even
    assert np.all((r.view(np.uint32) & 0xFFFF) == 0)
