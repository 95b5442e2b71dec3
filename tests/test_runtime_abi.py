"""The C-ABI library: builds, loads, exports what include/mtb200_rt.h declares, and
compiles kernels to sm_100a cubins without a GPU.  No launch happens here."""

import ctypes
import re
from pathlib import Path

import pytest

from mytriton_b200 import kernel_cases as cases
from mytriton_b200 import kernels as corpus
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


def test_cubin_cache_round_trip(runtime_lib, tmp_path, monkeypatch):
    """A kernel compiled once is revived from disk without calling NVRTC again."""
    monkeypatch.setenv("MYTRITON_B200_CACHE", str(tmp_path))
    src = 'extern "C" __global__ void cached_k(float* x) { x[threadIdx.x] += 1.0f; }'
    first = runtime_lib.load_or_compile(src, "cached_k", NVRTC_OPTIONS)
    files = list(tmp_path.glob("cached_k-*.cubin"))
    assert len(files) == 1 and files[0].read_bytes() == first.cubin()

    def no_nvrtc(*args, **kwargs):
        raise AssertionError("NVRTC must not run on a cache hit")

    real_call = runtime_lib.call
    monkeypatch.setattr(runtime_lib, "call",
                        lambda name, *a: no_nvrtc() if name == "mtb_compile" else real_call(name, *a))
    second = runtime_lib.load_or_compile(src, "cached_k", NVRTC_OPTIONS)
    assert second.cubin() == first.cubin()
    # different options or source -> different entry
    monkeypatch.setattr(runtime_lib, "call", real_call)
    runtime_lib.load_or_compile(src, "cached_k", REFERENCE_NVRTC_OPTIONS)
    assert len(list(tmp_path.glob("cached_k-*.cubin"))) == 2
    monkeypatch.setenv("MYTRITON_B200_CACHE", "0")
    assert runtime_lib.cache_directory() is None


def test_concurrent_compiles_and_thread_local_errors(runtime_lib):
    """ctypes releases the GIL around each call: compiles run in parallel, every thread gets
    its own module, and a failing thread reads its own kernel's diagnostics (the error text is
    thread-local)."""
    from concurrent.futures import ThreadPoolExecutor

    def work(index: int):
        if index % 2:
            try:
                runtime_lib.Module(f'extern "C" __global__ void bad{index}() {{ int x = ; }}', f"bad{index}",
                                   NVRTC_OPTIONS)
            except runtime_lib.RuntimeLibraryError as error:
                return "error", f"bad{index}" in str(error)
            return "error", False
        source = f'extern "C" __global__ void good{index}(float* x) {{ x[threadIdx.x] = {index}.0f; }}'
        module = runtime_lib.Module(source, f"good{index}", NVRTC_OPTIONS)
        return "ok", len(module.cubin()) > 0

    with ThreadPoolExecutor(max_workers=8) as pool:
        results = list(pool.map(work, range(16)))
    assert [kind for kind, _ in results] == ["ok", "error"] * 8
    assert all(flag for _, flag in results)
