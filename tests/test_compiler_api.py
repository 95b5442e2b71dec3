"""JIT-driver behaviour the reference's tests pin (tests/test_cuda_compiler.py:107-315,
tests/test_ast_runtime_loop.py:284-303), checked on this package: grid validation,
specialisation cache, independent result copies, compile-only host calls."""

import numpy as np
import pytest

from mytriton_b200 import kernels as corpus
import mytriton_b200.compiler as compiler
from mytriton_b200.ssa import SSAForRange


def count_traces(monkeypatch):
    calls = []
    real = compiler.trace

    def counting(*args, **kwargs):
        calls.append(1)
        return real(*args, **kwargs)

    monkeypatch.setattr(compiler, "trace", counting)
    return calls


def test_rejects_boolean_and_empty_grids():
    out = np.empty(1, dtype=np.float32)
    for grid in ((True,), (0,), (), (1, 1, 1, 1), (1.0,)):
        with pytest.raises(ValueError, match="invalid launch grid"):
            corpus.scalar_copy_kernel[grid](out, out)


def test_compilation_is_cached_across_grids_and_calls(monkeypatch):
    calls = count_traces(monkeypatch)
    corpus.tile_kernel.clear_cache()
    out = np.empty(64, dtype=np.float32)
    corpus.tile_kernel[(1,)](out, 64, TILE_SIZE=32)
    corpus.tile_kernel[(2,)](out, 64, TILE_SIZE=32)
    corpus.tile_kernel[lambda meta: (64 // meta["TILE_SIZE"],)](out, 33, TILE_SIZE=32)
    assert len(calls) == 1
    corpus.tile_kernel[(1,)](out, 64, TILE_SIZE=16)          # new constexpr value
    assert len(calls) == 2
    corpus.tile_kernel[(1,)](out, 64, TILE_SIZE=32, num_warps=1)   # backend knob is part of the key
    assert len(calls) == 3


def test_runtime_scalar_type_is_part_of_the_key(monkeypatch):
    calls = count_traces(monkeypatch)
    corpus.runtime_full_kernel.clear_cache()
    out = np.empty(8, dtype=np.float32)
    corpus.runtime_full_kernel[(1,)](out, 5, 3, BLOCK=8)
    corpus.runtime_full_kernel[(1,)](out, 5, 4, BLOCK=8)      # same types: hit
    corpus.runtime_full_kernel[(1,)](out, 5, 1.25, BLOCK=8)   # float fill: new specialisation
    assert len(calls) == 2


def test_constexpr_must_be_plain_values():
    out = np.empty(8, dtype=np.float32)
    with pytest.raises(TypeError, match="BLOCK: constexpr value must be bool, int, float, or str"):
        corpus.full_and_zeros_kernel[(1,)](out, 8, BLOCK=[8])


def test_arrays_are_validated_on_every_call():
    good = np.zeros(16, dtype=np.float32)
    corpus.compile_only_kernel[(1,)](good, good, good, 16, TILE=16)
    strided = np.zeros(32, dtype=np.float32)[::2]
    with pytest.raises(TypeError, match="only C-contiguous arrays are supported"):
        corpus.compile_only_kernel[(1,)](strided, good, good, 16, TILE=16)
    with pytest.raises(TypeError, match="only float32 arrays are supported"):
        corpus.compile_only_kernel[(1,)](good.astype(np.float64), good, good, 16, TILE=16)


def test_results_are_independent_copies():
    out = np.zeros(1, dtype=np.float32)
    corpus.nested_runtime_loops_kernel.clear_cache()
    ops, first_ssa, first_src = corpus.nested_runtime_loops_kernel[(1,)](out, 3)
    outer = next(op for op in first_ssa if isinstance(op, SSAForRange))
    outer.body.clear()
    ops.clear()
    again_ops, cached_ssa, cached_src = corpus.nested_runtime_loops_kernel[(1,)](out, 3)
    assert next(op for op in cached_ssa if isinstance(op, SSAForRange)).body
    assert again_ops and cached_src == first_src


def test_result_behaves_like_a_three_tuple():
    out = np.zeros(4, dtype=np.float32)
    result = corpus.nested_pointer_kernel[(1,)](out)
    assert isinstance(result, tuple) and len(result) == 3
    assert isinstance(result[0], list) and isinstance(result[1], list) and isinstance(result[2], str)
    assert "nested_pointer_kernel" in result[2]
    assert result == tuple(result)


def test_host_arguments_never_load_the_native_runtime(monkeypatch):
    import mytriton_b200.cuda_utils as cuda_utils

    def fail():
        raise AssertionError("the GPU runtime must not be touched for NumPy arguments")

    monkeypatch.setattr(cuda_utils, "_runtime", fail)
    x = np.ones(16, dtype=np.float32)
    corpus.compile_only_kernel.clear_cache()
    corpus.compile_only_kernel[(1,)](x, x, np.empty_like(x), 16, TILE=16)


def test_mlir_backend_is_refused(monkeypatch):
    monkeypatch.setenv("MYTRITON_BACKEND", "mlir")
    out = np.zeros(1, dtype=np.float32)
    with pytest.raises(ValueError, match="MLIR backend is not part of this build"):
        corpus.scalar_copy_kernel[(1,)](out, out)
    monkeypatch.setenv("MYTRITON_BACKEND", "metal")
    with pytest.raises(ValueError, match="unsupported backend"):
        corpus.scalar_copy_kernel[(1,)](out, out)
