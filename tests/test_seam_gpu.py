"""The two-call seam a maintainer of the reference would bind (code generator +
execute_cuda_if_needed), driven by hand the way src/mytriton/compiler.py:132-213 does."""

import inspect

import numpy as np
import pytest

from mytriton_b200 import kernels as corpus
from mytriton_b200 import device, runtime
from mytriton_b200.ast_frontend import trace
from mytriton_b200.cuda_codegen import SSACUDACodegen
from mytriton_b200.cuda_utils import execute_cuda_if_needed
from mytriton_b200.ssa import SSALowering
from mytriton_b200.ssa_verification import SSAVerifier

pytestmark = pytest.mark.gpu


def test_generate_then_execute_by_hand(gpu):
    n = 5000
    rng = np.random.default_rng(0)
    x = rng.standard_normal(n, dtype=np.float32)
    dx, dout = device.to_device(x), device.empty(n)
    kernel = corpus.sigmoid_kernel
    bound = kernel.signature.bind(dx, dout, n, BLOCK=1024)
    ops, params = trace(kernel.fn, kernel.signature, bound.arguments)
    ssa_ops = SSAVerifier(None).verify(SSALowering().lower(ops))
    codegen = SSACUDACodegen()
    artifact = codegen.generate_artifact("sigmoid_kernel", ssa_ops, params)
    assert codegen.generate("sigmoid_kernel", ssa_ops, params) == artifact.src
    cache: dict = {}
    for _ in range(2):                                   # second call hits the kernel cache
        execute_cuda_if_needed(
            kernel_cache=cache, cuda_src=artifact.src, kernel_name="sigmoid_kernel",
            launch_grid=(5,), threads_per_block=artifact.plan.threads,
            runtime_args=(dx, dout, n), plan=artifact.plan, param_names=("x", "out", "n"))
    runtime.synchronize()
    assert len(cache) == 1
    np.testing.assert_allclose(dout.to_host(), 1 / (1 + np.exp(-x)), rtol=1e-5, atol=1e-6)


def test_mixed_host_and_device_arrays_are_rejected(gpu):
    dx = device.empty(16)
    host = np.zeros(16, dtype=np.float32)
    with pytest.raises(TypeError, match="mixed NumPy and CuPy arrays"):
        corpus.compile_only_kernel[(1,)](dx, host, dx, 16, TILE=16)


def test_block_larger_than_the_device_limit_is_refused(gpu):
    dx = device.empty(16)
    with pytest.raises(ValueError, match="exceeds device limit"):
        execute_cuda_if_needed(
            kernel_cache={}, cuda_src='extern "C" __global__ void k(float* x) {}', kernel_name="k",
            launch_grid=(1,), threads_per_block=2048, runtime_args=(dx,))
    assert inspect.signature(execute_cuda_if_needed).parameters["kernel_cache"].kind.name == "KEYWORD_ONLY"
