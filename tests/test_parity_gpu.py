"""GPU parity: this backend vs the reference's generated kernels vs the CPU oracle.

Every case runs three ways on the same seeded inputs (see gpu_utils).  Outputs
*and* inputs are compared afterwards, so a stray write shows up as a mismatch.

Bars: elementwise / index / loop-arithmetic kernels are bit-exact against the
reference's kernels; reductions, softmax and matmuls agree with the reference's
kernels and the oracle within 1e-5 relative error (the summation order differs
by design).  Against the NumPy oracle ``exp`` differs from CUDA's ``expf`` in the
last ulp, so sigmoid/softmax use rtol 1e-5 / atol 1e-6 there, the tolerances of
the reference's own tests.
"""

import numpy as np
import pytest

from mytriton_b200 import kernel_cases as cases
import gpu_utils

pytestmark = pytest.mark.gpu

BIT_EXACT = [
    "add_1024", "add_256", "copy_256", "relu_256", "relu_1024", "leaky_relu_256",
    "leaky_relu_1024", "sigmoid_256", "sigmoid_1024", "matrix_add_256", "tile_shape_4x8",
    "matrix_add_2d_16x32", "two_carried", "annotated_carried", "no_carried",
    "sequential_loops", "nested_loops", "full_and_zeros", "runtime_full_int",
    "runtime_full_float", "tile_32", "scalar_copy", "nested_pointer", "nonzero_range",
    "compile_only", "extremum", "int_reduce_64", "int_reduce_1024", "where_minimum_256",
    "matrix_add_2d_6x10", "tile_shape_3x5", "add_48",
]
TOLERANT = [
    "row_sum_1024", "row_sum_8", "row_max_1024", "row_min_1024", "softmax_1024", "softmax_8",
    "softmax_1", "long_row_sum_static", "long_row_sum_loop_1024", "naive_matmul_k17",
    "matmul_2d_k5", "matmul_runtime_k", "matmul_runtime_k_4x8", "matmul_runtime_k_32x32",
    "softmax_64", "row_sum_2", "chunked_row_stats_256",
]
ORACLE_EXP_CASES = {"sigmoid_256", "sigmoid_1024", "softmax_1024", "softmax_8", "softmax_1"}


def _close(actual, expected, rtol, atol):
    np.testing.assert_allclose(actual, expected, rtol=rtol, atol=atol, equal_nan=True)


@pytest.mark.parametrize("name", BIT_EXACT)
def test_bit_exact_against_reference_kernel(name, golden, gpu):
    case = cases.CASES_BY_NAME[name]
    host = gpu_utils.seeded_arrays(case, specials=True)
    mine = gpu_utils.run_mine(case, host)
    theirs = gpu_utils.run_reference_source(case, golden[name], host)
    oracle = gpu_utils.run_oracle(case, golden[name]["ssa"], host)
    for index, (a, b, c) in enumerate(zip(mine, theirs, oracle)):
        if not isinstance(a, np.ndarray):
            continue
        assert gpu_utils.same_bits(a, b), f"{name}: array #{index} differs from the reference kernel"
        if name in ORACLE_EXP_CASES:
            _close(a, c, 1e-5, 1e-6)
        else:
            assert gpu_utils.same_values(a, c), f"{name}: array #{index} differs from the oracle"


@pytest.mark.parametrize("name", TOLERANT)
def test_reductions_and_matmuls_within_tolerance(name, golden, gpu):
    case = cases.CASES_BY_NAME[name]
    host = gpu_utils.seeded_arrays(case)
    mine = gpu_utils.run_mine(case, host)
    theirs = gpu_utils.run_reference_source(case, golden[name], host)
    oracle = gpu_utils.run_oracle(case, golden[name]["ssa"], host)
    for a, b, c in zip(mine, theirs, oracle):
        if isinstance(a, np.ndarray):
            _close(a, b, 1e-5, 1e-5)
            _close(a, c, 1e-5, 1e-5)


@pytest.mark.parametrize("options", [{}, {"online_softmax": True}, {"num_warps": 4}, {"num_warps": 32}])
def test_softmax_4096_columns(options, gpu):
    """Wider than the reference can compile (its CTA would need 4096 threads)."""
    from oracle import numpy_oracle

    case = cases.CASES_BY_NAME["softmax_4096"]
    host = gpu_utils.seeded_arrays(case)
    host[0] *= 5.0
    mine = gpu_utils.run_mine(case, host, **options)
    expected = numpy_oracle.softmax_f64(host[0])
    assert np.max(np.abs(mine[1] - expected) / np.maximum(expected, 1e-30)) < 1e-5 or \
        np.allclose(mine[1], expected, rtol=1e-5, atol=1e-9)
    assert gpu_utils.same_bits(mine[0], host[0])


def test_softmax_large_values_known_answer(gpu):
    """The rows of the reference's tests/test_softmax_kernel.py:241-257."""
    from oracle import numpy_oracle
    from mytriton_b200 import kernels as corpus
    from mytriton_b200 import device, runtime

    x = np.array(
        [[1000.0, 1001.0, 999.0, 998.0], [-1000.0, -999.0, -1001.0, -1002.0],
         [1234.0, 1234.0, 1233.0, 1232.0]], dtype=np.float32)
    for options in ({}, {"online_softmax": True}):
        dx, dout = device.to_device(x), device.empty(x.shape)
        corpus.softmax_kernel[(3,)](dx, dout, 4, BLOCK=4, **options)
        runtime.synchronize()
        _close(dout.to_host(), numpy_oracle.softmax(x), 1e-4, 1e-4)


def test_extremum_table(gpu):
    """NaN propagation and the sign of zero: tests/test_math_ops.py:270-291."""
    from mytriton_b200 import kernels as corpus
    from mytriton_b200 import device, runtime

    table = [(np.nan, 2.0), (2.0, np.nan), (0.0, -0.0), (-0.0, 0.0), (3.0, 2.0), (2.0, 3.0)]
    for lhs, rhs in table:
        hi, lo = device.empty(1), device.empty(1)
        corpus.extremum_kernel[(1,)](float(lhs), float(rhs), hi, lo)
        runtime.synchronize()
        for got, want in ((hi.to_host()[0], np.maximum(np.float32(lhs), np.float32(rhs))),
                          (lo.to_host()[0], np.minimum(np.float32(lhs), np.float32(rhs)))):
            if np.isnan(want):
                assert np.isnan(got)
            else:
                assert got == want and np.signbit(got) == np.signbit(want)


def test_exact_integer_matmul(gpu):
    """a = arange, b = arange: exact in fp32 (tests/test_ast_runtime_loop.py:489-504)."""
    from mytriton_b200 import kernels as corpus
    from mytriton_b200 import device, runtime

    M, N, K = 19, 23, 5
    a = np.arange(M * K, dtype=np.float32).reshape(M, K)
    b = np.arange(K * N, dtype=np.float32).reshape(K, N)
    da, db, dc = device.to_device(a), device.to_device(b), device.empty((M, N))
    corpus.matmul_runtime_k_kernel[(3, 2)](da, db, dc, M, N, K, BM=8, BN=16)
    runtime.synchronize()
    assert np.array_equal(dc.to_host(), a @ b)


@pytest.mark.parametrize("name,options", [
    ("add_256", {"num_warps": 1}), ("add_256", {"num_warps": 32}), ("add_1024", {"elems_per_thread": 2}),
    ("softmax_64", {"num_warps": 4}), ("softmax_8", {"num_warps": 2}), ("row_sum_1024", {"num_warps": 1}),
    ("row_max_1024", {"num_warps": 32}), ("matrix_add_2d_16x32", {"num_warps": 1}),
    ("matrix_add_2d_6x10", {"num_warps": 4}), ("chunked_row_stats_256", {"num_warps": 2}),
    ("long_row_sum_loop_1024", {"num_warps": 32}), ("int_reduce_64", {"num_warps": 4}),
    ("softmax_1024", {"min_ctas_per_sm": 8, "num_warps": 4}), ("softmax_1024", {"online_softmax": True}),
    ("matmul_runtime_k_32x32", {"num_warps": 2}),
])
def test_layout_options_do_not_change_results(name, options, golden, gpu):
    """CTA size, elements per thread and occupancy hints only change the layout: more
    threads than elements, one warp for a wide block, guarded slots — same numbers."""
    case = cases.CASES_BY_NAME[name]
    host = gpu_utils.seeded_arrays(case)
    mine = gpu_utils.run_mine(case, host, **options)
    theirs = gpu_utils.run_reference_source(case, golden[name], host)
    exact = name in BIT_EXACT
    for a, b in zip(mine, theirs):
        if isinstance(a, np.ndarray):
            if exact:
                assert gpu_utils.same_bits(a, b)
            else:
                _close(a, b, 1e-5, 1e-5)


LOOP_CASES = ["long_row_sum_loop_1024", "matmul_runtime_k", "matmul_runtime_k_4x8", "matmul_runtime_k_32x32",
              "two_carried", "annotated_carried", "no_carried", "sequential_loops", "nested_loops",
              "chunked_row_stats_256"]


@pytest.mark.parametrize("name", LOOP_CASES)
def test_loop_passes_do_not_change_a_bit(name, gpu):
    """Every kernel with a run-time loop, compiled with the loop-aware passes (fold, CSE, DCE inside
    bodies, loop-invariant motion — the default) and without them: the same bits come out."""
    import mytriton_b200.kernels as corpus

    case = cases.CASES_BY_NAME[name]
    host = gpu_utils.seeded_arrays(case)
    getattr(corpus, case.kernel).clear_cache()
    optimised = gpu_utils.run_mine(case, host)
    plain = gpu_utils.run_mine(case, host, loop_passes=False)
    for index, (a, b) in enumerate(zip(optimised, plain)):
        if isinstance(a, np.ndarray):
            assert gpu_utils.same_bits(a, b), f"{name}: array #{index} changes with the loop passes"
