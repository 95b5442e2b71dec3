"""Run-time if / else / not / return on the GPU against the closed forms of
tests/test_control_flow.py (elementwise part bit-exact; block sums to 1e-5 relative to the
sum of magnitudes, because the device adds in a different order)."""

import numpy as np
import pytest

import corpus
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
