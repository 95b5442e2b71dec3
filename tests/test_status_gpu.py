"""A device wait that runs out must come back as a status code, not as a hang or a trap.

The kernel below waits, with the GEMM kernel's own bounded-wait helper and a short
limit, on an mbarrier that nothing ever arrives on.  It must return within
microseconds, record its code in the status word, and leave the context usable."""

import ctypes

import numpy as np
import pytest

from mytriton_b200 import device, dot_codegen, runtime
from mytriton_b200.cuda_utils import NVRTC_OPTIONS

pytestmark = pytest.mark.gpu

KERNEL = r'''
extern "C" __global__ void starved_wait(unsigned* status, unsigned* reached_end) {
    __shared__ unsigned long long bar;
    __shared__ unsigned abort_word;
    if (threadIdx.x == 0) {
        abort_word = 0u;
        mtb_mbar_init(mtb_smem(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // parity 0 of a fresh barrier completes only after an arrival; none will come
    const bool ok = mtb_mbar_wait(mtb_smem(&bar), 0u, &abort_word, status, 0x77u);
    __syncthreads();
    if (threadIdx.x == 0) *reached_end = ok ? 1u : 2u;
}
'''


def test_wait_limit_sets_status_and_kernel_returns(gpu):
    src = "#define MTB_WAIT_LIMIT 200000ll\n" + dot_codegen._PRELUDE + KERNEL
    module = runtime.Module(src, "starved_wait", NVRTC_OPTIONS)
    status = device.DeviceArray((4,), "uint32").fill_u32(0)
    end = device.DeviceArray((4,), "uint32").fill_u32(0)
    module.launch((1,), (64,), [ctypes.c_uint64(status.ptr), ctypes.c_uint64(end.ptr)])
    runtime.synchronize()                                   # returns: the wait was bounded
    assert end.to_host()[0] == 2
    with pytest.raises(runtime.RuntimeLibraryError) as caught:
        runtime.status_check(status.ptr)
    assert caught.value.code == -6 and "0x00000077" in str(caught.value)
    # the context is still healthy: ordinary work runs afterwards
    x = device.to_device(np.arange(8, dtype=np.float32))
    assert np.array_equal(x.to_host(), np.arange(8, dtype=np.float32))


def test_a_reported_status_is_cleared_so_later_launches_check_clean(gpu):
    """check_status() reports a timed-out wait once and zeroes the device's status word: the
    next healthy launch must not fail on the old code."""
    word = dot_codegen.status_word(runtime)
    runtime.memset_u32(word, 0x31, 1)
    runtime.synchronize()
    with pytest.raises(runtime.RuntimeLibraryError):
        dot_codegen.check_status()
    dot_codegen.check_status()                              # clean again


def test_a_prepared_launch_runs_on_its_own_device_whatever_device_is_current(gpu):
    """A process that drives two GPUs: the module is loaded once per device, a prepared launch
    carries its device, and the caller's current device is left as it was."""
    if runtime.device_count() < 2:
        pytest.skip("needs two GPUs")
    from mytriton_b200 import kernels as corpus

    n = 4096
    host_x = np.arange(n, dtype=np.float32)
    host_y = np.full(n, 0.5, dtype=np.float32)
    runs, outs = [], []
    for index in (0, 1):
        runtime.set_device(index)
        x, y, out = device.to_device(host_x), device.to_device(host_y * (index + 1)), device.empty(n)
        runs.append(corpus.add_kernel.launcher((4,), x, y, out, n, BLOCK=1024))
        outs.append((out, x, y))
    runtime.set_device(0)
    runs[1]()                                               # device 1's buffers while device 0 is current
    runs[0]()
    assert runtime.current_device() == 0
    for index in (0, 1):
        runtime.set_device(index)
        runtime.synchronize()
        assert np.array_equal(outs[index][0].to_host(), host_x + host_y * (index + 1))
    runtime.set_device(0)
