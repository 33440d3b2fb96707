"""Build the sm_100a shared library in-tree: ``python fast-attnres_b200/build.py``.

One ``nvcc`` invocation compiles ``csrc/attnres_b200.cu`` (which includes the
kernel headers) into ``attnres/_lib/libattnres_b200.so``.  nvcc cross-compiles
for sm_100a, so no GPU is needed to build.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
SOURCES = [ROOT / "csrc" / "attnres_b200.cu"]
HEADERS = sorted((ROOT / "csrc").glob("*.cuh")) + [ROOT.parent / "include" / "attnres_b200.h"]
OUTPUT = ROOT / "attnres" / "_lib" / "libattnres_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the sm_100a library cannot be built")
    return found


def up_to_date() -> bool:
    if not OUTPUT.exists():
        return False
    built = OUTPUT.stat().st_mtime
    return all(path.stat().st_mtime <= built for path in [*SOURCES, *HEADERS, Path(__file__)])


def build(*, force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if any source is newer than it; return its path."""
    if not force and up_to_date():
        return OUTPUT
    OUTPUT.parent.mkdir(parents=True, exist_ok=True)
    # ptxas always reports registers and spills (shown only when asked for): the flag also
    # fixes the order in which it lays the kernels out, so every build of the same sources
    # gives the same binary whether or not the report is printed.
    command = [_nvcc(), *NVCC_FLAGS, "-Xptxas", "-v", *map(str, SOURCES), "-o", str(OUTPUT)]
    result = subprocess.run(command, capture_output=True, text=True)
    if verbose or result.returncode != 0:
        sys.stderr.write(result.stdout + result.stderr)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {result.returncode}")
    return OUTPUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
