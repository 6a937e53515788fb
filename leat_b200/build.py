"""Builds libleat_sampler.so in-tree for sm_100a with nvcc (run as `python -m leat_b200.build`)."""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
LIBRARY = CSRC / "libleat_sampler.so"
SOURCES = [CSRC / "leat_sampler.cu"]
HEADERS = [CSRC / "sampler_kernels.cuh", CSRC / "device_util.cuh", CSRC / "stream_ring.cuh",
           CSRC / "general_kernel.cuh", CSRC / "filter_path.cuh",
           CSRC.parent.parent / "include" / "leat_sampler.h"]  # fmt: skip
# -fmad=false: the CPU statement of the algorithm rounds every product and sum separately, and
# ids must match it bit for bit
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-fmad=false",
         "-shared", "-Xcompiler", "-fPIC", "-std=c++17"]  # fmt: skip


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: the sampler has no path without its CUDA library")
    return found


def stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    return any(p.stat().st_mtime > built for p in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIBRARY
    command = [nvcc(), *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(LIBRARY),
               *map(str, SOURCES)]  # fmt: skip
    done = subprocess.run(command, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(done.stderr)
    if done.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{done.stdout}\n{done.stderr}")
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
