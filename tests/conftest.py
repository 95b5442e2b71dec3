import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for path in (str(ROOT), str(ROOT / "tests")):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


@pytest.fixture(scope="session")
def golden():
    import json

    return json.loads((ROOT / "tests" / "golden" / "corpus_golden.json").read_text())


@pytest.fixture(scope="session")
def runtime_lib():
    """The built native runtime; building it is part of the CPU test-suite."""
    from mytriton_b200 import build, runtime

    build.build_runtime()
    runtime.library()
    return runtime


@pytest.fixture(scope="session")
def gpu(runtime_lib):
    if not runtime_lib.is_available():
        pytest.fail("no CUDA device: GPU tests must run on a B200 box (there is no CPU fallback)")
    runtime_lib.set_device(0)
    return runtime_lib
