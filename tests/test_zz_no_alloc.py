"""The allocation-free row sum (`mtb_long_row_sum_static`) against the regular one.

Some callers cannot allocate device memory while they run — they own a fixed pool, or
sit in a loop where an allocation's stall is not acceptable — so this entry point
keeps its scratch inside the library.  It must give exactly what `mtb_long_row_sum`
gives with caller-provided scratch, call after call.  This file is collected last on
purpose: a run that stops at the first failure has then already run everything else.
"""

import ctypes as C

import numpy as np
import pytest

from mytriton_b200 import device, ops, runtime

pytestmark = pytest.mark.gpu


def reference_sum(dx, rows, cols):
    out = device.empty(rows).fill_u32(0x7FC00000)
    need = ops.long_row_sum_scratch_bytes(rows, cols)
    scratch = device.DeviceArray(((need + 3) // 4,), "uint32")
    ops.long_row_sum(dx, out, rows, cols, scratch, need)
    runtime.synchronize()
    return out.to_host()


def static_sum_through_c_abi(dx, rows, cols):
    out = device.empty(rows).fill_u32(0x7FC00000)
    lib = runtime.library()
    code = lib.mtb_long_row_sum_static(C.c_uint64(dx.ptr), C.c_uint64(out.ptr), rows, cols, None)
    assert code == 0, lib.mtb_last_error().decode()
    runtime.synchronize()
    return out.to_host()


@pytest.mark.parametrize("shape", [(8, 1 << 20), (37, 100_003), (1024, 4096)])
def test_two_calls_in_a_row_match_the_regular_entry_point(shape, gpu):
    rows, cols = shape
    rng = np.random.default_rng(rows + cols)
    first = rng.random(shape, dtype=np.float32) * 2 - 1
    second = rng.standard_normal(shape, dtype=np.float32)
    for x in (first, second):                      # the second call reuses the built-in scratch
        dx = device.to_device(x)
        want = reference_sum(dx, rows, cols)
        got = static_sum_through_c_abi(dx, rows, cols)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        np.testing.assert_allclose(got, x.astype(np.float64).sum(axis=1), rtol=1e-5,
                                   atol=1e-5 * np.abs(x).sum(axis=1).max())


def test_sizes_beyond_the_built_in_scratch_are_refused(gpu):
    rows, cols = 5000, 64                          # more rows than ticket slots
    dx, out = device.empty((rows, cols)), device.empty(rows)
    with pytest.raises(runtime.RuntimeLibraryError, match="exceeds the built-in scratch") as caught:
        ops.long_row_sum_static(dx, out, rows, cols)
    assert caught.value.code == -7
    rows = 4096                                    # the largest size it accepts still works
    x = np.ones((rows, cols), dtype=np.float32)
    got = static_sum_through_c_abi(device.to_device(x), rows, cols)
    assert np.array_equal(got, np.full(rows, float(cols), dtype=np.float32))


def test_calls_after_the_first_leave_free_device_memory_unchanged(gpu):
    """The point of the entry point: once it has run on a device (the first use makes the
    driver load the library's image), further calls take no device memory at all."""
    rows, cols = 64, 50_000
    dx = device.to_device(np.ones((rows, cols), dtype=np.float32))
    out = device.empty(rows)
    lib = runtime.library()

    def call():
        code = lib.mtb_long_row_sum_static(C.c_uint64(dx.ptr), C.c_uint64(out.ptr), rows, cols, None)
        assert code == 0, lib.mtb_last_error().decode()

    call()                                         # set-up call
    runtime.synchronize()
    free_before, _ = runtime.mem_info()
    for _ in range(8):
        call()
    runtime.synchronize()
    free_after, _ = runtime.mem_info()
    assert free_after == free_before
    assert np.array_equal(out.to_host(), np.full(rows, float(cols), dtype=np.float32))
