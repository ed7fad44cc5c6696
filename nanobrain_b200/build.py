"""Builds the C-ABI shared library ``libnb_attn.so`` next to this package with nvcc for sm_100a.

The library is compiled in-tree (not into a JIT cache) so that the built file sits beside the
sources it came from. ``python -m nanobrain_b200.build`` rebuilds it.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libnb_attn.so"
SOURCES = [CSRC / "nb_attn.cu"]
HEADERS = sorted(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "nb_attn.h"]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-shared",
    "-Xcompiler",
    "-fPIC",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return nvcc


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(src.stat().st_mtime > built for src in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile ``libnb_attn.so`` if it is missing or older than its sources."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [find_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIB_PATH), *map(str, SOURCES)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
