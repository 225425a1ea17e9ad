"""In-tree build of ``libfss_b200.so`` (the C-ABI CUDA library) with plain nvcc for sm_100a.

No libtorch, no pybind: the only inputs are ``csrc/*.cu[h]`` and ``include/fss_b200.h``; the
result sits beside this file so that it travels with the source tree.  Run as
``python fast_sequential_scan_b200/build.py`` (add ``--force`` to rebuild, ``--verbose`` for ptxas
resource usage); run it as a script, not with ``-m``: importing the package needs the library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libfss_b200.so"

NVCC_FLAGS = [
    "-O3", "-std=c++17",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-shared",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: cannot build libfss_b200.so")
    return exe


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "fss_b200.h"]


def is_stale() -> bool:
    if not LIB.is_file():
        return True
    t = LIB.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources() + [Path(__file__)])


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not is_stale():
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIB)] + [str(f) for f in sorted(CSRC.glob("*.cu"))]
    env = dict(os.environ)
    res = subprocess.run(cmd, env=env, capture_output=True, text=True)
    if verbose or res.returncode:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode:
        raise RuntimeError("nvcc failed building libfss_b200.so")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
