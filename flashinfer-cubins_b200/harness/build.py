"""Builds ``lib/libnvfp4_b200.so`` from ``csrc/`` with nvcc for sm_100a.

The library is built in-tree (``python -m harness.build`` from the package root, or
``harness.build.build()``); nothing is compiled at run time. nvcc cross-compiles
without a GPU."""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_ROOT = Path(__file__).resolve().parents[1]
SOURCES = (PACKAGE_ROOT / "csrc" / "nvfp4_api.cu",)
HEADERS = tuple(sorted((PACKAGE_ROOT / "csrc").glob("*.cuh"))) + (
    PACKAGE_ROOT.parent / "include" / "nvfp4_b200.h",
)
OUTPUT = PACKAGE_ROOT / "lib" / "libnvfp4_b200.so"
FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "-cudart", "static",
)


def find_nvcc() -> str:
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise FileNotFoundError("nvcc not found; set NVCC")
    return nvcc


def is_current() -> bool:
    if not OUTPUT.is_file():
        return False
    built = OUTPUT.stat().st_mtime
    return all(path.stat().st_mtime <= built for path in (*SOURCES, *HEADERS))


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if a source is newer than it (or ``force``); returns its path."""
    if not force and is_current():
        return OUTPUT
    OUTPUT.parent.mkdir(parents=True, exist_ok=True)
    command = [find_nvcc(), *FLAGS, *(["-Xptxas", "-v"] if verbose else []),
               *map(str, SOURCES), "-o", str(OUTPUT)]
    result = subprocess.run(command, capture_output=True, text=True)
    if verbose or result.returncode:
        sys.stderr.write(result.stdout + result.stderr)
    if result.returncode:
        raise RuntimeError(f"nvcc failed with exit code {result.returncode}")
    return OUTPUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
