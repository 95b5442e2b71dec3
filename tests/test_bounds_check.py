"""The debug bounds-check mode: every global access is compared with its array's extent; an
access outside it is skipped and recorded, nothing traps.

The GPU cases never address memory outside an allocation: the extent handed to the kernel is made
*smaller* than the array really is (``extents=``), so the element the guard must protect is a
canary inside the buffer, and the run is safe whether or not the guard works."""

import numpy as np
import pytest

from mytriton_b200 import kernel_cases as cases
from mytriton_b200 import kernels as corpus
from mytriton_b200.cuda_utils import NVRTC_OPTIONS


def checked_source(name: str) -> str:
    case = cases.CASES_BY_NAME[name]
    kernel = getattr(corpus, case.kernel)
    return kernel[case.grid](*cases.build_args(case), **case.constexprs, bounds_check=True)[2]


@pytest.mark.parametrize("name", ["add_1024", "softmax_4096", "long_row_sum_loop_1024", "matmul_runtime_k_32x32",
                                  "scalar_copy", "matrix_add_2d_16x32", "chunked_row_stats_256"])
def test_every_access_goes_through_a_guard(name, runtime_lib):
    src = checked_source(name)
    case = cases.CASES_BY_NAME[name]
    body = src[src.index('extern "C"'):]
    assert "mtb_ck_ld(" in body or "mtb_ck_st(" in body
    assert "float4" not in body and "__ldcs" not in body and "__stcs" not in body    # element by element
    assert "long long mtb_ext_" in body and "unsigned* mtb_oob" in body
    # no raw subscript of a pointer parameter is left
    kernel = getattr(corpus, case.kernel)
    pointers = [line for line in body.splitlines()[1:2]][0]
    for token in pointers.split("(", 1)[1].split(","):
        token = token.strip()
        if token.startswith(("float*", "unsigned short*", "unsigned char*")):
            parameter = token.split()[-1]
            assert f"{parameter}[" not in body.split("{", 1)[1], parameter
    assert "__trap" not in src and "assert(" not in src
    runtime_lib.Module(src, case.kernel, NVRTC_OPTIONS)
    assert kernel is not None


def test_a_dot_kernel_stays_off_the_tensor_cores_when_checked():
    import ml_dtypes

    a = np.zeros((256, 128), ml_dtypes.bfloat16)
    b = np.zeros((128, 256), ml_dtypes.bfloat16)
    c = np.zeros((256, 256), np.float32)
    launcher = corpus.matmul_dot_kernel.launcher((2, 1), a, b, c, 256, 256, 128, BM=128, BN=256, BK=64,
                                                 bounds_check=True)
    assert launcher.artifact.plan.kind == "simt" and "mtb_ck_ld(" in launcher.artifact.src


@pytest.mark.gpu
def test_a_store_past_the_extent_is_skipped_and_reported(gpu):
    from mytriton_b200 import bounds, device, runtime

    n = 1000
    rng = np.random.default_rng(0)
    x, y = rng.random(n, dtype=np.float32), rng.random(n, dtype=np.float32)
    dx, dy = device.to_device(x), device.to_device(y)
    out = device.empty(n).fill_u32(0x7FC00000)
    bounds.check()                                           # starts clean
    # the kernel believes `out` has n - 1 elements; element n - 1 exists, but must stay untouched
    corpus.add_kernel[(4,)](dx, dy, out, n, BLOCK=256, bounds_check=True, extents={"out": n - 1})
    with pytest.raises(bounds.OutOfBoundsError) as caught:
        bounds.check(kernel=corpus.add_kernel)
    assert (caught.value.parameter, caught.value.index, caught.value.name) == (2, n - 1, "out")
    got = out.to_host()
    assert np.array_equal(got[:n - 1], (x + y)[:n - 1]) and np.isnan(got[n - 1])
    bounds.check()                                           # reported once, then clean
    with pytest.raises(ValueError, match="bounds_check=True"):
        corpus.add_kernel[(4,)](dx, dy, out, n, BLOCK=256, extents={"out": n - 1})
    # the context is healthy and an in-bounds run reports nothing
    out.fill_u32(0x7FC00000)
    corpus.add_kernel[(4,)](dx, dy, out, n, BLOCK=256, bounds_check=True)
    bounds.check()
    assert np.array_equal(out.to_host(), x + y)
    runtime.synchronize()


@pytest.mark.gpu
def test_a_load_past_the_extent_yields_zero_and_is_reported(gpu):
    from mytriton_b200 import bounds, device

    n = 512
    x = np.arange(1, n + 1, dtype=np.float32)
    y = np.full(n, 0.5, dtype=np.float32)
    dx, dy, out = device.to_device(x), device.to_device(y), device.empty(n)
    corpus.add_kernel[(2,)](dx, dy, out, n, BLOCK=256, bounds_check=True, extents={"x": n - 3})
    with pytest.raises(bounds.OutOfBoundsError) as caught:
        bounds.check(kernel=corpus.add_kernel)
    assert caught.value.name == "x" and n - 3 <= caught.value.index < n
    want = x + y
    want[n - 3:] = y[n - 3:]                                 # the skipped loads gave zero
    assert np.array_equal(out.to_host(), want)


@pytest.mark.gpu
def test_row_reduction_and_loop_kernels_run_checked(gpu):
    from mytriton_b200 import bounds, device

    rows, cols = 8, 4096
    rng = np.random.default_rng(1)
    m = rng.standard_normal((rows, cols), dtype=np.float32)
    dm, dp = device.to_device(m), device.empty((rows, cols))
    corpus.softmax_kernel[(rows,)](dm, dp, cols, BLOCK=4096, bounds_check=True)
    bounds.check()
    e = np.exp(m.astype(np.float64) - m.max(axis=1, keepdims=True))
    assert np.allclose(dp.to_host(), e / e.sum(axis=1, keepdims=True), rtol=1e-5, atol=1e-9)
    # the last row of the output is declared missing: its stores are skipped, the rest is right
    dp.fill_u32(0x7FC00000)
    corpus.softmax_kernel[(rows,)](dm, dp, cols, BLOCK=4096, bounds_check=True, extents={"out": (rows - 1) * cols})
    with pytest.raises(bounds.OutOfBoundsError) as caught:
        bounds.check(kernel=corpus.softmax_kernel)
    assert caught.value.parameter == 1 and caught.value.index >= (rows - 1) * cols
    got = dp.to_host()
    assert np.isnan(got[rows - 1]).all() and not np.isnan(got[:rows - 1]).any()
