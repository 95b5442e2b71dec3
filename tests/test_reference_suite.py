"""Runs the reference project's own test files against this package (CPU).

Only where a checkout of the reference sits next to this repository (directory
``reference`` beside the repository root); skipped anywhere else.  The reference's tests
import ``mytriton``; a small pytest plugin written to a temporary directory aliases that
name to this package, so the reference's test files run in place, unmodified.

Expected outcome: everything passes except (a) assertions on the exact text of the
reference's old one-thread-per-element CUDA source, which this backend replaces on
purpose, and (b) the MLIR backend, which is out of scope.  The failing set is pinned
below; any other failure — a front-end, SSA, verifier, optimiser or JIT-driver
difference — fails this test.
"""

import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REFERENCE_TESTS = ROOT.parent / "reference" / "tests"

PLUGIN = '''
import importlib, sys
sys.path.insert(0, {repo!r})
import mytriton_b200
sys.modules["mytriton"] = mytriton_b200
for name in ("language", "trace", "ast_frontend", "ssa", "type_inference", "ssa_verification",
             "optim", "cuda_codegen", "cuda_utils", "compiler", "block_shapes"):
    sys.modules["mytriton." + name] = importlib.import_module("mytriton_b200." + name)
'''

OLD_CUDA_TEXT = {          # assert the reference's generated source character by character
    "test_add_kernel.py::test_add_kernel_codegen[cuda]",
    "test_ast_runtime_loop.py::test_ast_frontend_lowers_runtime_range_to_cuda_for_loop",
    "test_ast_runtime_loop.py::test_nested_runtime_for_loops",
    "test_block_constructors.py::test_empty_lowers_to_uninitialized_cuda_value",
    "test_block_constructors.py::test_full_and_zeros_lowering_and_cuda_codegen",
    "test_copy_kernel.py::test_copy_kernel_codegen[cuda]",
    "test_cuda_compiler.py::test_nonzero_arange_start",
    "test_cuda_compiler.py::test_scalar_unmasked_load_and_store",
    "test_cuda_compiler.py::test_nested_pointer_arithmetic",
    "test_leaky_relu_kernel.py::test_leaky_relu_kernel_lowering",
    "test_long_row_sum_kernel.py::test_long_row_sum_kernel_lowering",
    "test_math_ops.py::test_extremum_lowering_and_cuda_codegen",
    "test_math_ops.py::test_unary_lowering_and_cuda_codegen",
    "test_math_ops.py::test_where_lowering_and_cuda_codegen",
    "test_math_ops.py::test_integer_extremum_does_not_emit_float_nan_checks",
    "test_matmul_2d_kernel.py::test_matmul_2d_generates_rank2_cuda_source_without_execution",
    "test_matrix_add_kernel.py::test_matrix_add_kernel",
    "test_naive_matmul_kernel.py::test_naive_matmul_kernel_lowering",
    "test_reduce_extremum_kernel.py::test_row_extremum_kernel_lowering",
    "test_reduce_sum_kernel.py::test_reduce_sum_kernel_lowering",
    "test_relu_kernel.py::test_relu_kernel_lowering",
    "test_sigmoid_kernel.py::test_sigmoid_kernel_lowering",
    "test_softmax_kernel.py::test_softmax_kernel_lowering",
    "test_tile_shape_kernel.py::test_matrix_add_2d_generates_cuda_for_degenerate_rank2_tiles",
    "test_tile_shape_kernel.py::test_matrix_add_2d_generates_rank2_cuda_source_without_execution",
}


def _allowed(test_id: str) -> bool:
    name = test_id.split("tests/")[-1]
    if "mlir" in name.lower():
        return True
    base = re.sub(r"\[.*$", "", name)
    return name in OLD_CUDA_TEXT or base in OLD_CUDA_TEXT


@pytest.mark.skipif(not REFERENCE_TESTS.is_dir(), reason="no checkout of the reference beside this repository")
def test_reference_test_files_pass_against_this_package(tmp_path):
    (tmp_path / "mytriton_alias_plugin.py").write_text(PLUGIN.format(repo=str(ROOT)))
    done = subprocess.run(
        [sys.executable, "-m", "pytest", str(REFERENCE_TESTS), "-p", "mytriton_alias_plugin",
         "-p", "no:cacheprovider", "-q", "--no-header", "-W", "ignore", "-rf",
         "--ignore", str(REFERENCE_TESTS / "test_mlir_codegen.py"),      # MLIR backend: out of scope
         "--rootdir", str(tmp_path), "-o", "cache_dir=" + str(tmp_path / "cache")],
        cwd=tmp_path, capture_output=True, text=True, timeout=600,
        env={"PYTHONPATH": str(tmp_path), "PATH": "/usr/bin:/bin", "HOME": str(tmp_path),
             "MYTRITON_B200_CACHE": "0"},
    )
    summary = done.stdout.strip().splitlines()[-1] if done.stdout.strip() else done.stderr[-400:]
    failed = [line.split(" - ")[0].removeprefix("FAILED ").strip()
              for line in done.stdout.splitlines() if line.startswith("FAILED ")]
    unexpected = [test_id for test_id in failed if not _allowed(test_id)]
    assert not unexpected, f"{summary}\nunexpected failures:\n" + "\n".join(unexpected)
    passed = int(re.search(r"(\d+) passed", summary).group(1))
    assert passed >= 135, summary
