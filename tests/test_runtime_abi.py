"""The C-ABI library: builds, loads, exports what include/mtb200_rt.h declares, and
compiles kernels to sm_100a cubins without a GPU.  No launch happens here."""

import ctypes
import re
from pathlib import Path

import pytest

import cases
import corpus
from mytriton_b200.cuda_utils import NVRTC_OPTIONS, REFERENCE_NVRTC_OPTIONS

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols() -> list[str]:
    header = (ROOT / "include" / "mtb200_rt.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    return sorted(set(re.findall(r"\b(mtb_[a-z0-9_]+)\s*\(", header)))


def test_header_and_binding_agree(runtime_lib):
    assert sorted(runtime_lib.EXPORTED_SYMBOLS) == declared_symbols()


def test_library_exports_every_declared_symbol(runtime_lib):
    lib = ctypes.CDLL(str(runtime_lib.LIBRARY_PATH))
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_compile_error_is_reported_not_raised_in_c(runtime_lib):
    with pytest.raises(runtime_lib.RuntimeLibraryError) as caught:
        runtime_lib.Module('extern "C" __global__ void k() { int x = ; }', "k", NVRTC_OPTIONS)
    assert caught.value.code == 200006          # NVRTC domain + NVRTC_ERROR_COMPILATION
    assert "expected an expression" in str(caught.value)


def test_bad_arguments_return_codes(runtime_lib):
    lib = runtime_lib.library()
    assert lib.mtb_compile(None, None, None, None, 0, None, None, 0) == -1
    assert b"NULL" in lib.mtb_last_error()
    assert lib.mtb_module_free(None) == 0


@pytest.mark.parametrize("case", [c for c in cases.CASES if c.expect_error is None],
                         ids=lambda c: c.name)
def test_generated_source_compiles_for_sm100a(case, runtime_lib):
    kernel = getattr(corpus, case.kernel)
    _, _, src = kernel[case.grid](*cases.build_args(case), **case.constexprs)
    module = runtime_lib.Module(src, case.kernel, NVRTC_OPTIONS)
    assert len(module.cubin()) > 0
    assert "warning" not in module.log.lower(), module.log


def test_reference_generated_sources_compile_with_reference_options(golden, runtime_lib):
    """What the GPU tests launch as "the reference's kernels" builds here too."""
    built = 0
    for name, entry in golden.items():
        if "cuda_src" in entry:
            runtime_lib.Module(entry["cuda_src"], entry["kernel"], REFERENCE_NVRTC_OPTIONS)
            built += 1
    assert built >= 35
