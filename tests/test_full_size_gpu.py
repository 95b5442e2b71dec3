"""Parity at the benchmark's full sizes.

The host cannot recompute these sizes in seconds, so each case is checked through
(a) the reference's own generated kernel on the same device where it can compile the
config (bit-exact for elementwise work), (b) fp64 NumPy on a seeded sample of rows or
elements, and (c) a size-independent property (softmax rows sum to one and are
invariant under a per-row shift; sums are linear; relu is idempotent)."""

import ctypes

import numpy as np
import pytest

from mytriton_b200 import kernel_cases as cases
from mytriton_b200 import kernels as corpus
import mytriton_b200 as triton
from mytriton_b200 import device, runtime
from mytriton_b200.cuda_utils import REFERENCE_NVRTC_OPTIONS
from oracle import numpy_oracle as no

pytestmark = pytest.mark.gpu


def reference_kernel(golden, case_name, grid, args):
    entry = golden[case_name]
    module = runtime.Module(entry["cuda_src"], entry["kernel"], REFERENCE_NVRTC_OPTIONS)
    packed = [ctypes.c_uint64(a.ptr) if isinstance(a, device.DeviceArray)
              else ctypes.c_int32(a) if isinstance(a, int) else ctypes.c_float(a) for a in args]
    module.launch(grid, (entry["threads_per_block"],), packed)
    runtime.synchronize()


@pytest.mark.parametrize("name,kernel,extra,case", [
    ("sigmoid", "sigmoid_kernel", (), "sigmoid_1024"),
    ("relu", "relu_kernel", (), "relu_1024"),
    ("leaky_relu", "leaky_relu_kernel", (0.01,), "leaky_relu_1024"),
])
def test_activations_on_2_to_28_elements(name, kernel, extra, case, golden, gpu):
    n = 2 ** 28
    rng = np.random.default_rng(1)
    x = rng.standard_normal(n, dtype=np.float32) * 2
    x[:6] = [np.nan, 0.0, -0.0, np.inf, -np.inf, -3.0]
    dx, mine, theirs = device.to_device(x), device.empty(n), device.empty(n)
    getattr(corpus, kernel)[(triton.cdiv(n, 2048),)](dx, mine, n, *extra, BLOCK=2048)
    reference_kernel(golden, case, (triton.cdiv(n, 1024),), [dx, theirs, n, *extra])
    runtime.synchronize()
    got, want = mine.to_host(), theirs.to_host()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))   # bit-exact, all 2^28
    sample = rng.choice(n, 1 << 16, replace=False)
    oracle = {"sigmoid": no.sigmoid, "relu": no.relu,
              "leaky_relu": lambda v: no.leaky_relu(v, 0.01)}[name](x[sample])
    np.testing.assert_allclose(got[sample], oracle, rtol=1e-5, atol=1e-6)
    if name == "relu":                                                  # idempotence
        again = device.empty(n)
        corpus.relu_kernel[(triton.cdiv(n, 2048),)](mine, again, n, BLOCK=2048)
        runtime.synchronize()
        assert np.array_equal(again.to_host().view(np.uint32), got.view(np.uint32))


def test_add_at_config_one_size(golden, gpu):
    case = cases.CASES_BY_NAME["add_1024"]
    n = 98_432
    rng = np.random.default_rng(0)
    x = rng.random(n, dtype=np.float32) * 2 - 1
    y = rng.random(n, dtype=np.float32) * 2 - 1
    dx, dy, mine, theirs = device.to_device(x), device.to_device(y), device.empty(n), device.empty(n)
    corpus.add_kernel[case.grid](dx, dy, mine, n, BLOCK=1024)
    reference_kernel(golden, "add_1024", case.grid, [dx, dy, theirs, n])
    runtime.synchronize()
    assert np.array_equal(mine.to_host(), no.add(x, y))
    assert np.array_equal(mine.to_host(), theirs.to_host())


@pytest.mark.parametrize("options", [{"num_warps": 4}, {"num_warps": 4, "online_softmax": True}])
def test_softmax_8192_by_4096(options, gpu):
    rows, cols = 8192, 4096
    rng = np.random.default_rng(2)
    x = rng.standard_normal((rows, cols), dtype=np.float32) * 5
    dx, dp = device.to_device(x), device.empty((rows, cols))
    corpus.softmax_kernel[(rows,)](dx, dp, cols, BLOCK=4096, **options)
    runtime.synchronize()
    p = dp.to_host()
    sample = rng.choice(rows, 256, replace=False)
    want = no.softmax_f64(x[sample])
    assert np.max(np.abs(p[sample] - want) / np.maximum(want, 1e-30)) < 1e-5
    np.testing.assert_allclose(p.sum(axis=1, dtype=np.float64), 1.0, rtol=0, atol=1e-5)
    # shift invariance: softmax(x + c_row) == softmax(x) up to the rounding of x + c
    shift = rng.integers(-8, 9, (rows, 1)).astype(np.float32)
    dshift, dq = device.to_device(x + shift), device.empty((rows, cols))
    corpus.softmax_kernel[(rows,)](dshift, dq, cols, BLOCK=4096, **options)
    runtime.synchronize()
    np.testing.assert_allclose(dq.to_host(), p, rtol=2e-5, atol=1e-9)


@pytest.mark.parametrize("kernel,oracle64", [
    ("row_sum_kernel", lambda x: x.astype(np.float64).sum(axis=1)),
    ("row_max_kernel", lambda x: x.max(axis=1).astype(np.float64)),
    ("row_min_kernel", lambda x: x.min(axis=1).astype(np.float64)),
])
def test_row_reductions_8192_by_4096(kernel, oracle64, gpu):
    rows, cols = 8192, 4096
    rng = np.random.default_rng(2)
    x = rng.standard_normal((rows, cols), dtype=np.float32) * 5
    dx, dout = device.to_device(x), device.empty(rows)
    getattr(corpus, kernel)[(rows,)](dx, dout, cols, BLOCK=4096)
    runtime.synchronize()
    got = dout.to_host()
    if kernel == "row_sum_kernel":
        assert no.reduction_relative_error(got, oracle64(x), x) < 1e-5
    else:
        assert np.array_equal(got.astype(np.float64), oracle64(x))        # extrema are exact


def test_long_row_sum_1024_by_2_to_20(gpu):
    rows, cols = 1024, 1 << 20
    rng = np.random.default_rng(3)
    dx = device.empty((rows, cols))
    sampled = {}
    chunk = 64                                              # generate and upload in row chunks
    for start in range(0, rows, chunk):
        block = rng.random((chunk, cols), dtype=np.float32) * 2 - 1
        runtime.memcpy_h2d(dx.ptr + start * cols * 4, block.ctypes.data, block.nbytes)
        runtime.synchronize()
        sampled[start] = (block[0].astype(np.float64).sum(), np.abs(block[0]).astype(np.float64).sum())
    dout = device.empty(rows)
    corpus.long_row_sum_loop_kernel[(rows,)](dx, dout, cols, BLOCK=2048, num_warps=16)
    runtime.synchronize()
    got = dout.to_host()
    for row, (want, scale) in sampled.items():
        assert abs(got[row] - want) / scale < 1e-5
    # linearity on the device: sum over both halves of every row equals the whole
    halves = device.empty(2 * rows)
    corpus.long_row_sum_loop_kernel[(2 * rows,)](dx, halves, cols // 2, BLOCK=2048, num_warps=16)
    runtime.synchronize()
    h = halves.to_host().astype(np.float64).reshape(rows, 2).sum(axis=1)
    np.testing.assert_allclose(h, got.astype(np.float64), rtol=0, atol=cols * 1e-5 * 0.5)
