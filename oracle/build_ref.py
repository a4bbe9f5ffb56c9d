"""Builds the reference-side checkers into oracle/_ref/ (git-ignored).  TEST INFRASTRUCTURE.

Compiles, from the reference's own sources where they lie (nothing is copied into this repository):
  * ref_function_base  -- this directory's driver + the reference's scheduler/kernel_key.hpp
  * scheduler_daemon   -- the reference's scheduler/scheduler_daemon.cpp, whose table loaders
                          (load_pair_eff / load_kernel_us, :230-264) accept or reject the emitted TSV files
If the reference tree is not present (the GPU box), nothing is built and the prebuilt files are used as they are.
"""
from __future__ import annotations

import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
# the reference checkout: KS_REFERENCE_DIR, or the directory "reference" beside this repository
REFERENCE = Path(os.environ.get("KS_REFERENCE_DIR") or HERE.parent.parent / "reference")


def build() -> bool:
    sched = REFERENCE / "scheduler"
    if not (sched / "kernel_key.hpp").exists():
        return False
    OUT.mkdir(exist_ok=True)
    jobs = [
        (OUT / "ref_function_base", ["g++", "-std=c++17", "-O2", "-I", str(sched), str(HERE / "ref_function_base_main.cpp")], [sched / "kernel_key.hpp", HERE / "ref_function_base_main.cpp"]),
        (OUT / "scheduler_daemon", ["g++", "-std=c++20", "-O2", "-w", str(sched / "scheduler_daemon.cpp"), "-lpthread", "-lrt"], [sched / "scheduler_daemon.cpp", sched / "shared_state.hpp"]),
    ]
    for target, cmd, deps in jobs:
        if target.exists() and all(target.stat().st_mtime >= d.stat().st_mtime for d in deps):
            continue
        subprocess.run(cmd + ["-o", str(target)], check=True)
    return True


if __name__ == "__main__":
    print("built" if build() else "reference tree not found: nothing built")
