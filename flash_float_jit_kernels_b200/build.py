"""In-tree build of the CUDA library (``csrc/libff_topk.so``) with nvcc.

The library is built for sm_100a only and kept beside its sources so the
loader (``_lib.py``) finds it without any JIT cache.  Run as
``python -m flash_float_jit_kernels_b200.build``.  The reference JIT-compiles
at first call instead (``jit_kernel/topk_indexer.py:76-106``).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
INCLUDE = Path(__file__).resolve().parent.parent / "include"
LIB_NAME = "libff_topk.so"
SOURCES = ["ff_topk.cu"]
HEADERS = ["ff_topk_common.cuh", "ff_topk_kernel.cuh", "ff_cp_exchange.cuh"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]


def lib_path() -> Path:
    return CSRC / LIB_NAME


def _nvcc() -> str:
    exe = shutil.which("nvcc")
    if exe is None:
        cand = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc"
        if cand.exists():
            exe = str(cand)
    if exe is None:
        raise RuntimeError("nvcc not found: cannot build libff_topk.so")
    return exe


def is_stale() -> bool:
    out = lib_path()
    if not out.exists():
        return True
    t = out.stat().st_mtime
    deps = [CSRC / s for s in SOURCES + HEADERS] + [INCLUDE / "ff_topk.h"]
    return any(d.stat().st_mtime > t for d in deps if d.exists())


def build_library(force: bool = False, verbose: bool = False, extra_flags=()) -> Path:
    """Compile ``csrc/*.cu`` into ``csrc/libff_topk.so`` (sm_100a)."""
    out = lib_path()
    if not force and not is_stale():
        return out
    cmd = [_nvcc(), *NVCC_FLAGS, *extra_flags]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(out)] + [str(CSRC / s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    return out


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
