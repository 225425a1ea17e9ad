"""Build recipe for the CPU checker libraries (test infrastructure, never shipped).

* ``oracle/libfss_oracle.so``  -- gcc build of ``scan_oracle.c`` (the C restatement).
* ``oracle/_ref/libfss_ref.so`` -- g++ build of ``ref_driver.cpp`` against the reference
  project's own header ``csrc/include/sequential_scan_cpu.hpp``, compiled where that header
  lies (``-I``), never copied.  Only built when the reference checkout is present; its
  location is ``$FSS_REFERENCE_DIR`` or the ``reference`` directory beside this repository.

* ``oracle/_ref/libfss_refgpu.so`` -- nvcc build of ``ref_gpu_driver.cu`` against the reference's
  own CUDA kernel headers (``csrc/include/sequential_scan_kernel[_bf16].cuh``), again by ``-I``,
  with the reference's flags (``-O3 --use_fast_math``, setup.py:17-19) but for sm_100a.  Used by the
  GPU parity tests and by the reference arm of the bench; only built when the reference and nvcc
  are present.

Run as ``python oracle/build_oracle.py``; ``__graft_entry__.build()`` calls :func:`build_all`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ORACLE_SO = HERE / "libfss_oracle.so"
REF_DIR = HERE / "_ref"
REF_SO = REF_DIR / "libfss_ref.so"
REF_GPU_SO = REF_DIR / "libfss_refgpu.so"


def reference_dir() -> Path | None:
    cand = os.environ.get("FSS_REFERENCE_DIR")
    path = Path(cand) if cand else HERE.parent.parent / "reference"
    header = path / "csrc" / "include" / "sequential_scan_cpu.hpp"
    return path if header.is_file() else None


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.is_file():
        return True
    t = target.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources)


def build_oracle(force: bool = False) -> Path:
    src = HERE / "scan_oracle.c"
    if force or _stale(ORACLE_SO, [src, Path(__file__)]):
        cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared",
               "-fvisibility=hidden", "-o", str(ORACLE_SO), str(src), "-lm"]
        subprocess.run(cmd, check=True)
    return ORACLE_SO


def build_ref(force: bool = False) -> Path | None:
    """Compile the reference's CPU loop; returns None when the reference is not present."""
    ref = reference_dir()
    if ref is None:
        return REF_SO if REF_SO.is_file() else None
    src = HERE / "ref_driver.cpp"
    hdr = ref / "csrc" / "include" / "sequential_scan_cpu.hpp"
    if force or _stale(REF_SO, [src, hdr, Path(__file__)]):
        REF_DIR.mkdir(exist_ok=True)
        # -O3 like the reference's own build (setup.py:17); no -fopenmp: its pragma is racy.
        cmd = ["g++", "-O3", "-ffp-contract=off", "-std=c++17", "-fPIC", "-shared", "-pthread",
               "-fvisibility=hidden", "-I", str(ref / "csrc" / "include"),
               "-o", str(REF_SO), str(src)]
        subprocess.run(cmd, check=True)
    return REF_SO


def build_ref_gpu(force: bool = False) -> Path | None:
    """Compile the reference's CUDA kernels behind a C ABI; None when the reference or nvcc is absent
    (a library built earlier is still returned: it travels with the tree)."""
    ref = reference_dir()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if ref is None or not Path(nvcc).exists():
        return REF_GPU_SO if REF_GPU_SO.is_file() else None
    src = HERE / "ref_gpu_driver.cu"
    inc = ref / "csrc" / "include"
    hdrs = [inc / "sequential_scan_kernel.cuh", inc / "sequential_scan_kernel_bf16.cuh"]
    if force or _stale(REF_GPU_SO, [src, *hdrs, Path(__file__)]):
        REF_DIR.mkdir(exist_ok=True)
        cmd = [nvcc, "-O3", "--use_fast_math", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
               "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared", "-I", str(inc),
               "-o", str(REF_GPU_SO), str(src)]
        subprocess.run(cmd, check=True)
    return REF_GPU_SO


def build_all(force: bool = False) -> dict:
    return {"oracle": build_oracle(force), "ref": build_ref(force), "ref_gpu": build_ref_gpu(force)}


if __name__ == "__main__":
    out = build_all(force="--force" in sys.argv)
    for k, v in out.items():
        print(f"{k}: {v}")
