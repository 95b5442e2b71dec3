"""The split-row sum (multi-CTA row reduction) through the C ABI."""

import numpy as np
import pytest

from mytriton_b200 import device, ops, runtime
from oracle import numpy_oracle as no

pytestmark = pytest.mark.gpu


def run(x: np.ndarray) -> np.ndarray:
    rows, cols = x.shape
    dx, dout = device.to_device(x), device.empty(rows).fill_u32(0x7FC00000)
    need = ops.long_row_sum_scratch_bytes(rows, cols)
    scratch = device.DeviceArray(((need + 3) // 4,), "uint32").fill_u32(0xDEADBEEF)
    ops.long_row_sum(dx, dout, rows, cols, scratch, need)
    ops.long_row_sum(dx, dout, rows, cols, scratch, need)      # tickets must be reusable
    runtime.synchronize()
    return dout.to_host()


@pytest.mark.parametrize("shape", [(8, 1 << 20), (3, 1_000_003), (1024, 4096), (31, 4097),
                                   (1, 5), (5, 1), (200, 65_536)])
def test_matches_fp64_sum_within_1e5(shape, gpu):
    rng = np.random.default_rng(shape[0] * 31 + shape[1])
    x = rng.random(shape, dtype=np.float32) * 2 - 1
    got = run(x)
    assert no.reduction_relative_error(got, no.row_sum_f64(x), x) < 1e-5


def test_is_deterministic(gpu):
    rng = np.random.default_rng(7)
    x = rng.standard_normal((6, 3_000_000), dtype=np.float32)
    assert np.array_equal(run(x).view(np.uint32), run(x).view(np.uint32))


def test_rejects_small_scratch_and_bad_sizes(gpu):
    dx, dout = device.empty((4, 8192)), device.empty(4)
    scratch = device.DeviceArray((4,), "uint32")
    with pytest.raises(runtime.RuntimeLibraryError, match="scratch too small"):
        ops.long_row_sum(dx, dout, 4, 8192, scratch, 16)
    with pytest.raises(runtime.RuntimeLibraryError, match="positive"):
        ops.long_row_sum_scratch_bytes(0, 10)

