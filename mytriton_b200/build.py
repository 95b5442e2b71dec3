"""Builds the native runtime (libmtb200.so) in-tree with nvcc for sm_100a."""

from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
REPO_ROOT = PACKAGE_DIR.parent
LIBRARY = PACKAGE_DIR / "libmtb200.so"
SOURCES = [PACKAGE_DIR / "csrc" / "mtb200_rt.cu", PACKAGE_DIR / "csrc" / "mtb200_rowsum.cu"]
HEADERS = [REPO_ROOT / "include" / "mtb200_rt.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O2", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def find_nvcc() -> str:
    candidate = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(candidate):
        raise RuntimeError("nvcc not found; the runtime library cannot be built")
    return candidate


def is_stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    return any(path.stat().st_mtime > built for path in (*SOURCES, *HEADERS) if path.exists())


def build_runtime(force: bool = False, verbose: bool = False) -> Path:
    """Compile csrc/*.cu into libmtb200.so next to this file; returns its path."""
    if not force and not is_stale():
        return LIBRARY
    command = [
        find_nvcc(), *NVCC_FLAGS, f"-I{REPO_ROOT / 'include'}",
        "-o", str(LIBRARY), *map(str, SOURCES), "-ldl",
    ]
    if verbose:
        print(" ".join(command))
    done = subprocess.run(command, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{done.stdout}\n{done.stderr}")
    return LIBRARY


if __name__ == "__main__":
    print(build_runtime(force=True, verbose=True))
