"""What the generated CUDA looks like (CPU): layouts, vectorisation decisions,
reduction shape, literals.  Complements the parity tests, which only see results."""

import numpy as np
import pytest

from mytriton_b200 import kernel_cases as cases
from mytriton_b200 import kernels as corpus
from mytriton_b200.cuda_codegen import SSACUDACodegen
from mytriton_b200.nodes import Const, Param, Store
from mytriton_b200.ssa import SSALowering
from mytriton_b200.trace import Value
from mytriton_b200.types import F32, I32, PTR_F32
import mytriton_b200 as triton
import mytriton_b200.language as tl


def source(name, **options):
    case = cases.CASES_BY_NAME[name]
    kernel = getattr(corpus, case.kernel)
    return kernel[case.grid](*cases.build_args(case), **case.constexprs, **options)[2]


def artifact(name, **options):
    case = cases.CASES_BY_NAME[name]
    kernel = getattr(corpus, case.kernel)
    return kernel.launcher(case.grid, *cases.build_args(case), **case.constexprs, **options).artifact


def test_float_literals_keep_the_reference_spelling():
    gen = SSACUDACodegen()
    assert gen.literal(float("nan")) == "__int_as_float(0x7fc00000)"
    assert gen.literal(float("inf")) == "__int_as_float(0x7f800000)"
    assert gen.literal(float("-inf")) == "(-__int_as_float(0x7f800000))"
    assert gen.literal(-0.0) == "-0.0f" and gen.literal(1.25) == "1.25f"
    assert gen.literal(True) == "true" and gen.literal(7) == "7"


def test_cta_size_is_decoupled_from_block_size():
    assert artifact("add_1024").plan.threads == 128              # 8 elements per thread
    assert artifact("softmax_4096").plan.threads == 512          # the reference needs 4096 threads
    assert artifact("softmax_4096", num_warps=4).plan.threads == 128
    assert artifact("two_carried").plan.threads == 1             # scalar kernel
    assert artifact("nonzero_range").plan.threads == 4           # tiny blocks: one thread per element
    assert artifact("add_1024").plan.notes["layouts"] == {"1024": {"regs": 8, "vec": 4}}


def test_contiguous_accesses_are_128_bit_and_streaming():
    src = source("add_1024")
    assert src.count("__ldcs(reinterpret_cast<const float4*>") == 2
    assert src.count("__stcs(reinterpret_cast<float4*>") == 1
    assert "& 15ull) == 0ull" in src                              # run-time alignment test
    assert "x[v" in src                                           # scalar path for the ragged edge


def test_row_stride_times_runtime_scalar_still_vectorises_along_the_row():
    src = source("matrix_add_2d_16x32")                           # offs_m * N + offs_n
    assert "float4" in src


def test_column_vector_loads_are_not_vectorised():
    src = source("matmul_runtime_k_32x32")                        # a[offs_m * K + k]: stride K along rows
    body = src.split("for (int v", 1)[1]
    assert "float4" not in body.split("}", 1)[0]


def test_reductions_use_shuffles_and_one_barrier():
    src = source("row_sum_1024")
    assert "__shfl_xor_sync(0xffffffffu" in src
    assert src.count("__syncthreads()") == 1
    assert "__shared__ float red_" in src and "[4];" in src       # one slot per warp (128 threads)
    assert source("row_sum_8").count("__syncthreads()") == 0      # a single partial warp


def test_online_softmax_fuses_the_two_reductions():
    two_pass = source("softmax_4096")
    fused = source("softmax_4096", online_softmax=True)
    assert two_pass.count("__syncthreads()") == 2
    assert fused.count("__syncthreads()") == 1 and "float2 osm_" in fused


def test_extremum_expression_matches_the_reference_form():
    value, out = Param("value", F32), Param("out", PTR_F32)
    ssa = SSALowering().lower([Store(out, tl.maximum(Value(value), 2.0).expr, None)])
    src = SSACUDACodegen().generate("extremum", ssa, [value, out])
    assert ("(isnan(value) ? (value) : (isnan(2.0f) ? (2.0f) : "
            "((value) > (2.0f) ? (value) : (2.0f))))") in src
    ints = SSALowering().lower([Store(out, tl.minimum(Value(Param("n", I32)), 2).expr, None)])
    assert "isnan" not in SSACUDACodegen().generate("m", ints, [Param("n", I32), out])


def test_loop_carried_block_lives_in_registers():
    src = source("long_row_sum_loop_1024")
    assert "for (int v" in src and "float v" in src
    assert src.count("__syncthreads()") == 1                      # only the final reduction


def test_register_held_value_used_in_another_shape_goes_through_shared_memory(runtime_lib):
    """A loop-carried vector broadcast over a tile after the loop: its registers are in the
    vector's own layout, so it is redistributed through shared memory (the result itself is
    checked on the GPU by the attention test)."""
    from mytriton_b200.cuda_utils import NVRTC_OPTIONS
    from mytriton_b200.ssa import SSAPrinter
    from oracle import ssa_interp

    @triton.jit
    def carried_then_broadcast(out, n):
        acc = tl.zeros((8,), tl.float32)
        for k in range(n):
            acc = acc + 1.0
        tl.store(out + tl.arange(0, 4)[:, None] * 8 + tl.arange(0, 8)[None, :], acc[None, :])

    out = np.zeros(32, np.float32)
    _, ssa_ops, src = carried_then_broadcast[(1,)](out, 3)
    assert "__shared__ float cvt_" in src
    runtime_lib.Module(src, "carried_then_broadcast", NVRTC_OPTIONS)
    ssa_interp.run(SSAPrinter().print_ops(ssa_ops), {"out": out, "n": 3}, (1,))
    assert np.all(out == 3.0)


@triton.jit
def mixed_extremum_kernel(x, out, n, BLOCK: tl.constexpr):
    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
    mask = offs < n
    a = tl.load(x + offs, mask=mask, other=0.0)
    tl.store(out + offs, tl.minimum(offs, 1.5) + tl.maximum(a, n), mask=mask)


def test_mixed_int_float_extremum_converts_the_integer_operand(runtime_lib):
    """isnan() on an int is ambiguous to NVRTC: the integer side of a mixed maximum or
    minimum is converted to float before the NaN tests (the reference's text does not
    compile for this kernel)."""
    from mytriton_b200.cuda_utils import NVRTC_OPTIONS

    x = np.zeros(64, np.float32)
    _, _, src = mixed_extremum_kernel[(1,)](x, x, 64, BLOCK=64)
    assert "isnan((float)(" in src
    runtime_lib.Module(src, "mixed_extremum_kernel", NVRTC_OPTIONS)


@triton.jit
def ticket_wait_kernel(flag, x, out, n, limit, BLOCK: tl.constexpr):
    """Takes a ticket with a scalar atomic, then polls the flag word (a scalar load inside a
    ``while``) with a block reduction in the loop body: every thread of the CTA must see the same
    flag value on every iteration, or the reduction's barrier would be reached by part of it."""
    lanes = tl.arange(0, BLOCK)
    tl.atomic_add(flag, 1.0)
    seen = tl.load(flag)
    spins = n * 0
    total = 0.0
    while (seen < limit) & (spins < 4):
        total = total + tl.sum(tl.load(x + lanes, mask=lanes < n, other=0.0))
        seen = tl.load(flag)
        spins = spins + 1
    tl.store(out, total)


def test_scalar_loads_are_read_once_per_cta_and_broadcast(runtime_lib):
    """One thread reads a scalar (volatile), the CTA gets it through shared memory between two
    barriers; a scalar store or atomic is followed by a barrier.  The kernel is compiled, not run:
    a kernel that spins on another program's flag is not something to launch in a test."""
    from mytriton_b200.cuda_utils import NVRTC_OPTIONS

    flag = np.zeros(1, np.float32)
    _, _, src = ticket_wait_kernel[(2,)](flag, np.zeros(256, np.float32), np.zeros(1, np.float32), 256, 2.0, BLOCK=256)
    lines = [line.strip() for line in src.splitlines()]
    reads = [i for i, line in enumerate(lines) if "(volatile float*)flag" in line]
    assert len(reads) == 2
    for i in reads:
        assert lines[i].startswith("if (threadIdx.x == 0) { uni_")
        assert lines[i - 1] == "__syncthreads();" and lines[i + 1] == "__syncthreads();"
        assert lines[i + 2].startswith("float v") and lines[i + 2].endswith(lines[i].split()[5] + ";")
    atomic = next(i for i, line in enumerate(lines) if "atomicAdd(&flag[0]" in line)
    assert lines[atomic].startswith("if (threadIdx.x == 0)") and lines[atomic + 1] == "__syncthreads();"
    # the loop leaves on a value that came through the broadcast slot
    leave = next(i for i, line in enumerate(lines) if line.startswith("if (!(") and line.endswith("break;"))
    assert leave > reads[0]
    runtime_lib.Module(src, "ticket_wait_kernel", NVRTC_OPTIONS)
