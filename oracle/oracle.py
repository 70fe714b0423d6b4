"""CPU oracle for the top-k indexer -- TEST INFRASTRUCTURE ONLY.

Used by ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline /
reference arm of ``bench.py`` as the checker; the product package never
imports it.

Three independent statements of the same contract
(``jit_kernel/topk_indexer.py:109-152``; short rows
``jit_kernel/csrc/topk_indexer/topk_indexer_radix.cu:180-191``; window slicing
``benchmark/bench_topk.py:132-148``):

* :func:`topk_stable_sort` -- ``torch.sort(descending=True, stable=True)`` per
  window, the definition named as the reference result;
* :func:`topk_numpy` -- numpy argsort on the composite (monotone key, index);
* :func:`topk_c` -- ``oracle_topk.c`` through ctypes (quickselect + sort).

Pinning: all three are checked against the golden vectors under
``tests/golden`` (``tests/test_oracle.py``).  The reference has no golden
vectors for this path and its kernel needs a GPU, so parity with the reference
kernel's exact outputs is unpinned; the stable-sort definition is pinned.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path
from typing import Optional

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
_LIB_PATH = HERE / "liboracle_topk.so"


# --------------------------------------------------------------------------
# statement 1: torch stable sort
# --------------------------------------------------------------------------
def topk_stable_sort(score: torch.Tensor, lengths: torch.Tensor, k: int,
                     row_starts: Optional[torch.Tensor] = None) -> torch.Tensor:
    score = score.detach().cpu()
    lengths = lengths.detach().cpu()
    B, L = score.shape
    out = torch.full((B, k), -1, dtype=torch.int32)
    for b in range(B):
        rs = int(row_starts[b]) if row_starts is not None else 0
        n = max(0, min(int(lengths[b]), L - rs))
        if n <= k:
            out[b, :n] = torch.arange(n, dtype=torch.int32)
            continue
        win = score[b, rs:rs + n]
        order = torch.sort(win, descending=True, stable=True).indices
        out[b] = order[:k].to(torch.int32)
    return out


# --------------------------------------------------------------------------
# statement 2: numpy on composite keys
# --------------------------------------------------------------------------
def monotone_key(x: np.ndarray) -> np.ndarray:
    """Order-preserving fp32 -> uint32 map with -0.0 == +0.0 and NaN on top."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).copy()
    a = u & np.uint32(0x7FFFFFFF)
    u[a == 0] = 0
    neg = (u >> np.uint32(31)).astype(bool)
    key = np.where(neg, ~u, u | np.uint32(0x80000000)).astype(np.uint32)
    key[a > np.uint32(0x7F800000)] = np.uint32(0xFFFFFFFF)
    return key


def topk_numpy(score: np.ndarray, lengths: np.ndarray, k: int,
               row_starts: Optional[np.ndarray] = None) -> np.ndarray:
    score = np.asarray(score, dtype=np.float32)
    B, L = score.shape
    out = np.full((B, k), -1, dtype=np.int32)
    for b in range(B):
        rs = int(row_starts[b]) if row_starts is not None else 0
        n = max(0, min(int(lengths[b]), L - rs))
        if n <= k:
            out[b, :n] = np.arange(n, dtype=np.int32)
            continue
        key = monotone_key(score[b, rs:rs + n]).astype(np.uint64)
        comp = (key << np.uint64(32)) | (~np.arange(n, dtype=np.uint32)).astype(np.uint64)
        top = np.argpartition(comp, n - k)[n - k:]
        top = top[np.argsort(comp[top])[::-1]]
        out[b] = top.astype(np.int32)
    return out


# --------------------------------------------------------------------------
# statement 3: the C restatement
# --------------------------------------------------------------------------
def build_c(force: bool = False) -> Path:
    src = HERE / "oracle_topk.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["gcc", "-O2", "-fPIC", "-std=c11", "-ffp-contract=off", "-shared", "-o", str(_LIB_PATH),
                        str(src), "-lm"], check=True)
    return _LIB_PATH


_clib = None


def _c():
    global _clib
    if _clib is None:
        lib = ctypes.CDLL(str(build_c()))
        i32p = ctypes.c_void_p
        lib.oracle_topk_transform.restype = ctypes.c_int
        lib.oracle_topk_transform.argtypes = [
            ctypes.c_void_p, ctypes.c_int64, i32p, i32p, i32p, ctypes.c_int32, ctypes.c_int64,
            ctypes.c_int32, ctypes.c_int32, i32p, ctypes.c_int64, i32p, ctypes.c_int32, i32p]
        lib.oracle_indexer_logits.restype = ctypes.c_int
        lib.oracle_indexer_logits.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                              ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64)]
        lib.oracle_key_of_bits.restype = ctypes.c_uint32
        lib.oracle_key_of_bits.argtypes = [ctypes.c_uint32]
        _clib = lib
    return _clib


def _np_ptr(a):
    return None if a is None else a.ctypes.data


def topk_c(score: np.ndarray, lengths: np.ndarray, k: int, row_starts=None, *, epilogue: int = 0,
           table=None, cu_seqlens_q=None, offsets=None) -> np.ndarray:
    score = np.asarray(score, dtype=np.float32)
    assert score.ndim == 2 and score.strides[1] == 4
    B, L = score.shape
    lengths = np.ascontiguousarray(lengths, dtype=np.int32)
    rs = None if row_starts is None else np.ascontiguousarray(row_starts, dtype=np.int32)
    tb = None if table is None else np.ascontiguousarray(table, dtype=np.int32)
    cu = None if cu_seqlens_q is None else np.ascontiguousarray(cu_seqlens_q, dtype=np.int32)
    of = None if offsets is None else np.ascontiguousarray(offsets, dtype=np.int32)
    out = np.empty((B, k), dtype=np.int32)
    rc = _c().oracle_topk_transform(
        score.ctypes.data, score.strides[0] // 4, _np_ptr(lengths), _np_ptr(rs), out.ctypes.data,
        B, L, k, epilogue, _np_ptr(tb), 0 if tb is None else tb.shape[1], _np_ptr(cu),
        0 if cu is None else len(cu) - 1, _np_ptr(of))
    if rc != 0:
        raise RuntimeError(f"oracle_topk_transform failed: {rc}")
    return out


def key_c(bits: int) -> int:
    return int(_c().oracle_key_of_bits(bits & 0xFFFFFFFF))


# --------------------------------------------------------------------------
# epilogues and context-parallel pieces (pure Python/numpy statements)
# --------------------------------------------------------------------------
def transform_page_table(idx: np.ndarray, src_page_table: np.ndarray,
                         cu_seqlens_q: Optional[np.ndarray]) -> np.ndarray:
    """dst[i, j] = src[r(i), idx[i, j]] (topk_indexer_radix.cu:1000-1085)."""
    B, k = idx.shape
    out = np.full((B, k), -1, dtype=np.int32)
    for b in range(B):
        r = b
        if cu_seqlens_q is not None:
            r = next(q for q in range(len(cu_seqlens_q) - 1)
                     if cu_seqlens_q[q] <= b < cu_seqlens_q[q + 1])
        v = idx[b] >= 0
        out[b, v] = src_page_table[r, idx[b, v]]
    return out


def transform_ragged(idx: np.ndarray, offsets: np.ndarray) -> np.ndarray:
    """out[i, j] = idx[i, j] + offsets[i] (topk_indexer_radix.cu:1087-1124)."""
    out = idx.copy()
    for b in range(idx.shape[0]):
        v = idx[b] >= 0
        out[b, v] = idx[b, v] + offsets[b]
    return out


def cp_local(score_shard: np.ndarray, lengths: np.ndarray, k: int, shard_offset: int):
    """Shard-local candidates: (value bits as int32 [B,k], global index [B,k])."""
    B, Lw = score_shard.shape
    loc = np.clip(lengths.astype(np.int64) - shard_offset, 0, Lw).astype(np.int32)
    idx = topk_numpy(score_shard, loc, k)
    for b in range(B):          # a shard shorter than k still emits its run in canonical order
        n = int(loc[b])
        if 0 < n <= k:
            key = monotone_key(score_shard[b, :n]).astype(np.uint64)
            comp = (key << np.uint64(32)) | (~np.arange(n, dtype=np.uint32)).astype(np.uint64)
            idx[b, :n] = np.argsort(comp)[::-1].astype(np.int32)
    val = np.full((B, k), -np.inf, dtype=np.float32)
    gidx = np.full((B, k), -1, dtype=np.int32)
    for b in range(B):
        v = idx[b] >= 0
        val[b, v] = score_shard[b, idx[b, v]]
        gidx[b, v] = idx[b, v] + shard_offset
    return val, gidx


def cp_merge(cand_val: np.ndarray, cand_idx: np.ndarray, lengths: np.ndarray, k: int) -> np.ndarray:
    """cand_* are [P, B, k]; exact merge under (value desc, global index asc)."""
    P, B, _ = cand_val.shape
    out = np.full((B, k), -1, dtype=np.int32)
    for b in range(B):
        n = int(lengths[b])
        if n <= k:
            out[b, :max(n, 0)] = np.arange(max(n, 0), dtype=np.int32)
            continue
        v = cand_val[:, b, :].reshape(-1)
        g = cand_idx[:, b, :].reshape(-1)
        ok = g >= 0
        v, g = v[ok], g[ok]
        key = monotone_key(v).astype(np.uint64)
        comp = (key << np.uint64(32)) | (~g.astype(np.uint32)).astype(np.uint64)
        order = np.argsort(comp)[::-1][:k]
        out[b, :len(order)] = g[order]
    return out


def indexer_logits(q: np.ndarray, k: np.ndarray, w: np.ndarray):
    """One row of lightning-indexer logits: q [64, 128], k [n, 128] (fp8 e4m3 values widened to
    float32), w [64] -> (scores float32 [n], number of dot products not exact in float32)."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    assert q.shape == (64, 128) and k.ndim == 2 and k.shape[1] == 128 and w.shape == (64,)
    out = np.empty(k.shape[0], dtype=np.float32)
    bad = ctypes.c_int64(0)
    rc = _c().oracle_indexer_logits(q.ctypes.data, k.ctypes.data, w.ctypes.data, k.shape[0], out.ctypes.data,
                                    ctypes.byref(bad))
    if rc != 0:
        raise RuntimeError(f"oracle_indexer_logits failed: {rc}")
    return out, int(bad.value)
