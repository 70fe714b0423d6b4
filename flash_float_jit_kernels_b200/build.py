"""In-tree build of the CUDA libraries (``csrc/libff_topk.so`` and
``csrc/libff_indexer.so``) with nvcc.

The libraries are built for sm_100a only and kept beside their sources so the
loaders (``_lib.py``, ``indexer_logits.py``) find them without any JIT cache.  Run as
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
INDEXER_LIB_NAME = "libff_indexer.so"      # the logit producer: its own library and header
INDEXER_SOURCES = ["ff_indexer_logits.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]


def lib_path() -> Path:
    flags = env_flags()
    if not flags:
        return CSRC / LIB_NAME
    return CSRC / LIB_NAME.replace(".so", _knob_suffix(flags) + ".so")


def indexer_lib_path() -> Path:
    return CSRC / INDEXER_LIB_NAME


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


def env_flags():
    """Compile-time knobs taken from the environment, as ``-D`` flags (the reference does the same
    with its ``FLASH_FLOAT_TOPK_*`` variables, ``jit_kernel/topk_indexer.py:11-48``):
    ``FF_TOPK_TILE_UNITS`` (16-byte units per shared-memory tile, a multiple of 512 up to 4096) and
    ``FF_TOPK_EXTRA_NVCC_FLAGS`` (anything else, space separated).  A library built with knobs gets
    them into its file name, so that it never replaces the default build."""
    flags = []
    tile = os.environ.get("FF_TOPK_TILE_UNITS")
    if tile:
        flags.append(f"-DFF_TOPK_TILE_UNITS={int(tile)}")
    flags += os.environ.get("FF_TOPK_EXTRA_NVCC_FLAGS", "").split()
    return flags


def _knob_suffix(flags) -> str:
    import hashlib
    return "" if not flags else "_" + hashlib.sha1(" ".join(flags).encode()).hexdigest()[:8]


def _compile(out: Path, sources, verbose: bool, extra_flags) -> Path:
    cmd = [_nvcc(), *NVCC_FLAGS, *extra_flags]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(out)] + [str(CSRC / s) for s in sources]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    return out


def build_library(force: bool = False, verbose: bool = False, extra_flags=()) -> Path:
    """Compile ``csrc/ff_topk.cu`` into ``csrc/libff_topk.so`` (sm_100a)."""
    out = lib_path()
    if not force and not is_stale():
        return out
    return _compile(out, SOURCES, verbose, [*env_flags(), *extra_flags])


CHECKED_LIB_NAME = "libff_topk_checked.so"   # the same library compiled with -DFF_BOUNDS_CHECK


def checked_lib_path() -> Path:
    return CSRC / CHECKED_LIB_NAME


def build_checked_library(force: bool = False, verbose: bool = False) -> Path:
    """``csrc/libff_topk_checked.so``: ``ff_topk.cu`` with ``-DFF_BOUNDS_CHECK``, in which every
    data-dependent index into a work array is range-checked and a violation sets
    ``FF_STATUS_BOUNDS`` in the status word instead of touching memory (a debugging build;
    the product loads ``libff_topk.so``)."""
    out = checked_lib_path()
    deps = [CSRC / s for s in SOURCES + HEADERS] + [INCLUDE / "ff_topk.h"]
    if not force and out.exists() and all(d.stat().st_mtime <= out.stat().st_mtime for d in deps if d.exists()):
        return out
    return _compile(out, SOURCES, verbose, ["-DFF_BOUNDS_CHECK"])


def build_indexer_library(force: bool = False, verbose: bool = False, extra_flags=()) -> Path:
    """Compile ``csrc/ff_indexer_logits.cu`` into ``csrc/libff_indexer.so`` (sm_100a)."""
    out = indexer_lib_path()
    deps = [CSRC / s for s in INDEXER_SOURCES] + [INCLUDE / "ff_indexer_logits.h"]
    if not force and out.exists() and all(d.stat().st_mtime <= out.stat().st_mtime for d in deps):
        return out
    return _compile(out, INDEXER_SOURCES, verbose, extra_flags)


TVMFFI_LIB_NAME = "libff_topk_tvmffi.so"   # the reference's own FFI symbol, forwarding to libff_topk.so


def tvmffi_lib_path() -> Path:
    return CSRC / TVMFFI_LIB_NAME


def build_tvmffi_module(force: bool = False) -> Path:
    """Compile ``csrc/ff_topk_tvm_ffi.cc`` (host code, g++) into ``csrc/libff_topk_tvmffi.so``: a
    TVM-FFI module exporting ``fast_topk`` as the reference's wrapper calls it
    (``jit_kernel/topk_indexer.py:141-149``).  Needs the ``tvm_ffi`` package (headers and library)."""
    import tvm_ffi.libinfo as li
    out = tvmffi_lib_path()
    src = CSRC / "ff_topk_tvm_ffi.cc"
    deps = [src, INCLUDE / "ff_topk.h"]
    if not force and out.exists() and all(d.stat().st_mtime <= out.stat().st_mtime for d in deps):
        return out
    build_library()
    tvm_lib = Path(li.find_libtvm_ffi())
    cxx = shutil.which("g++") or "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-o", str(out), str(src),
           f"-I{li.find_include_path()}", f"-I{li.find_dlpack_include_path()}",
           f"-L{CSRC}", "-l:" + LIB_NAME, f"-L{tvm_lib.parent}", "-ltvm_ffi",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tvm_lib.parent}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("g++ failed:\n" + res.stdout + res.stderr)
    return out


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_indexer_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_tvmffi_module(force="--force" in sys.argv))
    if "--checked" in sys.argv:
        print(build_checked_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
