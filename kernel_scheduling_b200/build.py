"""Builds libks_b200.so in-tree with nvcc for sm_100a (no GPU needed: nvcc cross-compiles).

    python -m kernel_scheduling_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libks_b200.so"
SOURCES = [CSRC / "ks_api.cu", CSRC / "ks_names.cpp", CSRC / "ks_pairtab.cpp", CSRC / "ks_synth.cpp"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-fmad=false",  # the float tables are defined as single IEEE operations: no contraction
    "-Xcompiler", "-fPIC", "-Xcompiler", "-pthread", "-shared",
    "--expt-relaxed-constexpr",
    "-ldl",  # NCCL is bound at run time (dlopen)
    "-lrt",  # shm_open (the shared-memory pair table)
]


def _stale() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.glob("*")) + [PKG.parent / "include" / "ks_b200.h"])
    return newest > LIB.stat().st_mtime


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libks_b200.so cannot be built")
    cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(LIB), *map(str, SOURCES)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode:
        raise RuntimeError("nvcc failed: " + " ".join(cmd))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
