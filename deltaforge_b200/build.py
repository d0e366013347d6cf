"""Build ``libdfb200.so`` in-tree with nvcc for sm_100a.

``python -m deltaforge_b200.build`` (or ``__graft_entry__.build()``) compiles every ``.cu`` under
``csrc/`` into one shared library next to this file. nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
# DFB200_BOUNDS_BUILD=1 (or `python -m deltaforge_b200.build --bounds`) selects the variant compiled with -DDFB_BOUNDS,
# whose kernels check their store and tile indices and report through the status word instead of making a bad access
BOUNDS = os.environ.get("DFB200_BOUNDS_BUILD") == "1" or "--bounds" in sys.argv
LIB = PKG / ("libdfb200_bounds.so" if BOUNDS else "libdfb200.so")
STAMP = PKG / (LIB.name + ".stamp")

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "-shared",
    *(["-DDFB_BOUNDS"] if BOUNDS else []),
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _fingerprint() -> str:
    h = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [PKG.parent / "include" / "dfb200.h"]):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    return LIB.exists() and STAMP.exists() and STAMP.read_text().strip() == _fingerprint()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library unless an up-to-date one is already there. Returns its path."""
    if not force and is_current():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libdfb200.so cannot be built on this machine")
    # Several processes (the ranks of one torchrun job) may find a stale library at the same moment: one of them
    # compiles, into a temporary file that replaces the library atomically, the others wait on the lock and then
    # find the stamp current.
    with open(PKG / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and is_current():
            return LIB
        tmp = PKG / f".libdfb200.{os.getpid()}.so.tmp"
        cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), *map(str, sources()), "-o", str(tmp)]
        proc = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
        if proc.returncode != 0:
            tmp.unlink(missing_ok=True)
            raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
        if verbose:
            print(proc.stderr)
        os.replace(tmp, LIB)
        STAMP.write_text(_fingerprint())
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
