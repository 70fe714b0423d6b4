"""Lightning-indexer logits: the producer of the scores ``fast_topk_v3`` selects from.

``scores[b, j] = sum_h w[b, h] * relu(q[b, h, :] . k[b, j, :])`` with 64 heads,
head_dim 128, q and K in fp8 e4m3 and fp32 accumulation, computed on the
Blackwell tensor cores (``csrc/ff_indexer_logits.cu``, C ABI in
``include/ff_indexer_logits.h``).  The reference has no such kernel; the shape is
the one its README names for the indexer (``README.md:28``).  There is no CPU
path: the loader raises if ``libff_indexer.so`` is missing.
"""
from __future__ import annotations

import ctypes
import functools
from ctypes import c_char_p, c_int, c_int32, c_int64, c_void_p
from typing import Optional

import torch

from .build import indexer_lib_path
from ._lib import LibraryMissingError
from .topk_indexer import TopkArgumentError, _ptr, _require, _stream_ptr

HEADS = 64
HEAD_DIM = 128

SIGNATURES = {
    "ff_indexer_logits_launch": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int32, c_int32,
         c_void_p, c_void_p],
    ),
    "ff_indexer_logits_launch_handover": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int32, c_int32,
         c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "ff_indexer_launch_count": (c_int64, []),
    "ff_indexer_last_error_string": (c_char_p, []),
}


@functools.lru_cache(maxsize=None)
def load() -> ctypes.CDLL:
    path = indexer_lib_path()
    if not path.exists():
        raise LibraryMissingError(
            f"{path} is missing: build it with `python -m flash_float_jit_kernels_b200.build` (there is no fallback)")
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


def new_handover(B: int, device) -> torch.Tensor:
    """A zero-filled survivor hand-over buffer for ``B`` rows (see :func:`indexer_topk`)."""
    from . import _lib
    return torch.zeros(B * _lib.FF_TOPK_HANDOVER_ROW_BYTES, dtype=torch.uint8, device=device)


def _check_handover(handover, threshold_hint, B, device):
    from . import _lib
    _require(threshold_hint is not None, "a hand-over buffer needs threshold_hint (the guesses the lists are built with)")
    _require(handover.dtype == torch.uint8 and handover.is_contiguous() and handover.device == device
             and handover.numel() >= B * _lib.FF_TOPK_HANDOVER_ROW_BYTES,
             "handover must be a contiguous uint8 tensor from new_handover(B, device)")
    _require(threshold_hint.shape == (B,) and threshold_hint.dtype == torch.float32 and threshold_hint.is_contiguous()
             and threshold_hint.device == device, "threshold_hint must be a contiguous (B) float32 tensor")


def indexer_logits_fp8(q: torch.Tensor, k: torch.Tensor, w: torch.Tensor, lengths: torch.Tensor, *,
                       out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
                       ctas_per_row: int = 0, threshold_hint: Optional[torch.Tensor] = None,
                       handover: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Scores of every key of every row.

    With ``handover`` (from :func:`new_handover`) and ``threshold_hint`` the kernel also lists, per
    row, every score not below the row's guess for the select that follows
    (``fast_topk_v3(..., threshold_hint=..., handover=...)``), which then reads no score at all
    when the guess fits.

    Args:
        q: (B, 64, 128) ``float8_e4m3fn`` (or uint8 holding those bytes), contiguous.
        k: (B, L, 128) fp8 keys; ``stride(2) == 1``, ``stride(1) == 128``, any row stride that is
            a multiple of 16 bytes.
        w: (B, 64) float32 head weights.
        lengths: (B) int32 valid keys per row.
        out: optional (B, L) float32 result, ``stride(1) == 1``.
    Returns:
        (B, L) float32; positions ``>= lengths[b]`` that fall into a processed 128-key tile hold
        ``-inf``, later ones keep what ``out`` held (a fresh result is filled with ``-inf``).
    """
    _require(q.is_cuda and k.is_cuda and w.is_cuda and lengths.is_cuda, "all tensors must be CUDA tensors")
    _require(q.element_size() == 1 and k.element_size() == 1, "q and k must be fp8 (one byte per element)")
    _require(q.dim() == 3 and q.shape[1:] == (HEADS, HEAD_DIM) and q.is_contiguous(), "q must be contiguous [B, 64, 128]")
    B = q.size(0)
    _require(k.dim() == 3 and k.size(0) == B and k.size(2) == HEAD_DIM and k.stride(2) == 1
             and k.stride(1) == HEAD_DIM, "k must be [B, L, 128] with contiguous keys")
    L = k.size(1)
    _require(w.shape == (B, HEADS) and w.dtype == torch.float32 and w.is_contiguous(), "w must be contiguous float32 [B, 64]")
    _require(lengths.shape == (B,) and lengths.dtype == torch.int32 and lengths.is_contiguous(),
             "lengths must be contiguous int32 [B]")
    if out is None:
        out = torch.full((B, L), float("-inf"), dtype=torch.float32, device=q.device)
    else:
        _require(out.shape == (B, L) and out.dtype == torch.float32 and out.stride(1) == 1 and out.device == q.device,
                 "out must be float32 [B, L] with unit inner stride")
    if B == 0 or L == 0:
        return out
    lib = load()
    if handover is not None:
        _check_handover(handover, threshold_hint, B, q.device)
    with torch.cuda.device(q.device):
        rc = lib.ff_indexer_logits_launch_handover(
            q.data_ptr(), k.data_ptr(), k.stride(0) if B > 1 else max(k.stride(0), L * HEAD_DIM), w.data_ptr(),
            lengths.data_ptr(), out.data_ptr(), out.stride(0) if B > 1 else max(out.stride(0), L), B, L,
            int(ctas_per_row), None if handover is None else threshold_hint.data_ptr(), _ptr(handover),
            _ptr(status), _stream_ptr(q.device))
    if rc < 0:
        raise TopkArgumentError(f"indexer_logits_fp8: {lib.ff_indexer_last_error_string().decode()}")
    if rc > 0:
        raise RuntimeError(f"indexer_logits_fp8: {lib.ff_indexer_last_error_string().decode()}")
    return out


def indexer_topk(q: torch.Tensor, k: torch.Tensor, w: torch.Tensor, lengths: torch.Tensor, topk: int, *,
                 scores: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                 threshold_hint: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
                 handover: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One decode step of the indexer: logits from the fp8 K cache, then their top-k.

    Two launches on the current stream (producer, select), no host synchronisation; pass
    ``scores`` (B, L) float32, ``out`` (B, topk) int32 and, to carry threshold guesses from
    step to step, ``threshold_hint`` (see ``fast_topk_v3``) to keep the step allocation-free.
    With ``handover`` (:func:`new_handover`, kept from step to step like the guesses) the producer
    hands the select its survivors: every score not below a row's guess is listed while the scores
    are written, and a row whose guess fits is ranked from that list without reading a score.
    Returns the (B, topk) int32 indices; the result is exact with or without guesses and lists.
    """
    from .topk_indexer import fast_topk_v3
    scores = indexer_logits_fp8(q, k, w, lengths, out=scores, status=status,
                                threshold_hint=threshold_hint if handover is not None else None, handover=handover)
    return fast_topk_v3(scores, lengths, topk, out=out, status=status, threshold_hint=threshold_hint, handover=handover)
