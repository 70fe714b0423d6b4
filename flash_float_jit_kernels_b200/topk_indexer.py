"""Python operator layer of the top-k indexer.

Mirrors ``jit_kernel/topk_indexer.py:109-152`` (``fast_topk_v3``) and the
pybind entry points ``fast_topk_transform_fused`` /
``fast_topk_transform_ragged_fused``
(``jit_kernel/csrc/topk_indexer/topk_indexer_radix.cu:1549-1645``) of the
reference: same names, argument meaning and error behaviour.  PyTorch is used
for device memory and the current stream only; all work happens in the CUDA
library behind ``include/ff_topk.h``.

Result definition: for row ``i`` the window
``score[i, row_starts[i] : row_starts[i] + lengths[i]]`` is ranked by
(value descending, index ascending) and the first ``topk`` window-relative
positions are returned in that order; ``-0.0 == +0.0``; NaN ranks above
``+inf``.  Rows with ``lengths[i] <= topk`` return ``0..lengths[i]-1`` then
``-1`` (``topk_indexer_radix.cu:180-191``).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib


class TopkArgumentError(AssertionError, ValueError):
    """Bad operator arguments.

    The reference signals these with ``assert`` (``topk_indexer.py:132-135``)
    or ``TORCH_CHECK``; deriving from both lets either style of caller catch it.
    """


_WORKSPACES: dict = {}


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise TopkArgumentError(msg)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream_ptr(device: torch.device):
    return torch.cuda.current_stream(device).cuda_stream


def _workspace(lib, device: torch.device, B: int, L: int, k: int, stream: Optional[int] = None):
    """Per-(device, stream) scratch, grown on demand and zero-filled once."""
    need = int(lib.ff_topk_workspace_bytes(B, L, k))
    if need == 0:
        return None, 0
    key = (device.index, torch.cuda.current_stream(device).cuda_stream if stream is None else stream)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(need, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws, ws.numel()


_SCORE_DTYPES = {torch.float32: _lib.FF_DTYPE_F32, torch.bfloat16: _lib.FF_DTYPE_BF16, torch.float16: _lib.FF_DTYPE_F16}


def _check_common(score, lengths, topk, row_starts, dtypes=(torch.float32,)):
    _require(isinstance(topk, int) and 1 <= topk <= _lib.FF_TOPK_MAX_K,
             f"fast_topk_v3 supports topk in [1, {_lib.FF_TOPK_MAX_K}], got {topk}")
    _require(score.dim() == 2, "score must be 2-D [B, L]")
    _require(score.dtype in dtypes, "score must be " + " or ".join(str(d).replace("torch.", "") for d in dtypes))
    _require(score.is_cuda, "score must be a CUDA tensor (there is no CPU path)")
    _require(score.size(1) == 0 or score.stride(1) == 1, "score.stride(1) must be 1")
    B = score.size(0)
    _require(lengths.dim() == 1 and lengths.is_contiguous() and lengths.size(0) == B,
             "lengths must be a contiguous [B] tensor")
    _require(lengths.dtype == torch.int32, "lengths must be int32")
    _require(lengths.device == score.device, "lengths must live on score's device")
    if row_starts is not None:
        _require(row_starts.dim() == 1 and row_starts.size(0) == B and row_starts.is_contiguous(),
                 "row_starts must be a contiguous [B] tensor")
        _require(row_starts.dtype == torch.int32, "row_starts must be int32")
        _require(row_starts.device == score.device, "row_starts must live on score's device")


def fast_topk_v3(
    score: torch.Tensor,
    lengths: torch.Tensor,
    topk: int,
    row_starts: Optional[torch.Tensor] = None,
    *,
    out: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
    threshold_hint: Optional[torch.Tensor] = None,
    index_dtype: torch.dtype = torch.int32,
    handover: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Top-k indices of every row of ``score`` (reference: ``topk_indexer.py:109``).

    Args:
        score: (B, L) float32 CUDA tensor, ``stride(1) == 1``, any row stride.  bfloat16 and
            float16 scores are accepted as well (extension; the reference is fp32 only): each
            value is widened to fp32 exactly, so the result is that of the fp32 row with the
            same values, and half the bytes are read.
        lengths: (B) int32 valid length per row.
        topk: number of indices per row, 1..2048 (the reference accepts
            512, 1024 and 2048 only).
        row_starts: optional (B) int32 window start per row; returned indices
            are relative to the window.
        out: optional preallocated (B, topk) int32 or int64 result (extension; lets a
            caller keep the call allocation-free inside a CUDA graph).
        index_dtype: ``torch.int32`` (default, as the reference) or ``torch.int64`` (the
            layout ``torch.topk`` returns) for the result when ``out`` is not given.
        status: optional int32 device scalar that collects soft-error bits.
        threshold_hint: optional (B) float32 device tensor, read AND updated
            (extension; see :func:`new_threshold_hint`).  Entry ``i`` is a guess
            of a score between row ``i``'s k-th and 4096-th largest, NaN for "no
            guess".  A row with a fitting guess is swept once instead of twice
            and skips the histogram exchange; a guess that does not fit costs one
            extra sweep (``FF_STATUS_HINT_MISSED`` in ``status``).  The result
            is the same exact top-k either way.  On return the entry holds a
            score of rank about 1.25 k of this call's row: pass the tensor again
            for the next call on similar rows (the next decode step).

        handover: optional survivor lists written by the kernel that produced ``score`` with the
            same ``threshold_hint`` (``indexer_logits.indexer_logits_fp8(..., handover=...)``):
            a row whose guess fits is ranked from its list and no score is read; fp32 scores
            and int32 indices only.

    Returns:
        (B, topk) int32 indices in (value desc, index asc) order, ``-1``
        padded for rows shorter than ``topk``.
    """
    _check_common(score, lengths, topk, row_starts, dtypes=tuple(_SCORE_DTYPES))
    lib = _lib.load()
    B, L = score.size(0), score.size(1)
    if out is None:
        _require(index_dtype in (torch.int32, torch.int64), "index_dtype must be torch.int32 or torch.int64")
        out = torch.empty((B, topk), dtype=index_dtype, device=score.device)
    else:
        _require(out.shape == (B, topk) and out.dtype in (torch.int32, torch.int64) and out.is_contiguous()
                 and out.device == score.device, "out must be a contiguous (B, topk) int32 or int64 tensor")
    typed = score.dtype != torch.float32 or out.dtype != torch.int32
    if B == 0:
        return out
    dev = score.device
    stream = torch.cuda.current_stream(dev).cuda_stream
    ws, ws_bytes = _workspace(lib, dev, B, L, topk, stream)
    row_stride = score.stride(0) if B > 1 else max(score.stride(0), L)
    if threshold_hint is not None:
        _require(threshold_hint.shape == (B,) and threshold_hint.dtype == torch.float32
                 and threshold_hint.is_contiguous() and threshold_hint.device == dev,
                 "threshold_hint must be a contiguous (B) float32 tensor on score's device")

    if handover is not None:
        _require(not typed and threshold_hint is not None, "handover needs fp32 scores, int32 indices and threshold_hint")
        _require(handover.dtype == torch.uint8 and handover.is_contiguous() and handover.device == dev
                 and handover.numel() >= B * _lib.FF_TOPK_HANDOVER_ROW_BYTES,
                 "handover must be a contiguous uint8 tensor of B * FF_TOPK_HANDOVER_ROW_BYTES bytes")

    def call():
        if handover is not None:
            return lib.ff_topk_launch_handover(
                score.data_ptr(), row_stride, lengths.data_ptr(), _ptr(row_starts), out.data_ptr(), B, L, topk,
                threshold_hint.data_ptr(), threshold_hint.data_ptr(), handover.data_ptr(), _ptr(ws), ws_bytes,
                _ptr(status), stream)
        if typed:
            hint_ptr = None if threshold_hint is None else threshold_hint.data_ptr()
            return lib.ff_topk_launch_typed(
                score.data_ptr(), _SCORE_DTYPES[score.dtype], row_stride, lengths.data_ptr(), _ptr(row_starts),
                out.data_ptr(), 64 if out.dtype == torch.int64 else 32, B, L, topk, hint_ptr, hint_ptr,
                _ptr(ws), ws_bytes, _ptr(status), stream)
        if threshold_hint is None:
            return lib.ff_topk_launch(
                score.data_ptr(), row_stride, lengths.data_ptr(), _ptr(row_starts), out.data_ptr(), B, L, topk,
                _ptr(ws), ws_bytes, _ptr(status), stream)
        return lib.ff_topk_launch_hinted(
            score.data_ptr(), row_stride, lengths.data_ptr(), _ptr(row_starts), out.data_ptr(), B, L, topk,
            threshold_hint.data_ptr(), threshold_hint.data_ptr(), _ptr(ws), ws_bytes, _ptr(status), stream)

    # the library launches on the current device: switch only when score lives elsewhere
    if torch.cuda.current_device() == dev.index:
        rc = call()
    else:
        with torch.cuda.device(dev):
            rc = call()
    _lib.check(rc, "fast_topk_v3")
    return out


def new_threshold_hint(B: int, device) -> torch.Tensor:
    """A (B) float32 tensor of NaN ("no guess yet") for ``fast_topk_v3(threshold_hint=...)``."""
    return torch.full((B,), float("nan"), dtype=torch.float32, device=device)


def fast_topk_transform_fused(
    score: torch.Tensor,
    lengths: torch.Tensor,
    dst_page_table: torch.Tensor,
    src_page_table: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    row_starts: Optional[torch.Tensor] = None,
) -> None:
    """Top-k followed by a page-table gather, written into ``dst_page_table``.

    Mirrors ``fast_topk_transform_interface`` (``topk_indexer_radix.cu:1549-1600``):
    ``dst[i, j] = src_page_table[r(i), idx[i, j]]`` where ``r(i) = i`` in decode
    (``row_starts is None`` and one request per row) and otherwise the request
    whose ``cu_seqlens_q`` interval contains row ``i``.  ``k`` is
    ``dst_page_table.size(1)`` (the reference fixes it to 2048).
    """
    _require(dst_page_table.dim() == 2 and dst_page_table.is_contiguous(),
             "dst_page_table must be contiguous 2-D")
    topk = int(dst_page_table.size(1))
    _check_common(score, lengths, topk, row_starts)
    B, L = score.size(0), score.size(1)
    _require(dst_page_table.dtype == torch.int32 and src_page_table.dtype == torch.int32,
             "page tables must be int32")
    _require(src_page_table.dim() == 2 and src_page_table.stride(1) == 1,
             "src_page_table must be 2-D with unit inner stride")
    _require(cu_seqlens_q.dim() == 1 and cu_seqlens_q.is_contiguous()
             and cu_seqlens_q.dtype == torch.int32, "cu_seqlens_q must be contiguous int32 1-D")
    prefill_bs = cu_seqlens_q.size(0) - 1
    _require(dst_page_table.size(0) == B, "dst_page_table.size(0) must equal B")
    _require(src_page_table.size(0) == prefill_bs, "src_page_table.size(0) must equal len(cu_seqlens_q)-1")
    _require(prefill_bs <= B, "prefill batch must not exceed the expanded batch")
    if B == 0:
        return
    lib = _lib.load()
    is_decode = row_starts is None and prefill_bs == B
    ws, ws_bytes = _workspace(lib, score.device, B, L, topk)
    with torch.cuda.device(score.device):
        rc = lib.ff_topk_transform_launch(
            score.data_ptr(), score.stride(0) if B > 1 else max(score.stride(0), L),
            lengths.data_ptr(), _ptr(row_starts), dst_page_table.data_ptr(), B, L, topk,
            _lib.FF_EPILOGUE_PAGE_TABLE, src_page_table.data_ptr(), src_page_table.stride(0),
            None if is_decode else cu_seqlens_q.data_ptr(), prefill_bs, None,
            _ptr(ws), ws_bytes, None, _stream_ptr(score.device))
    _lib.check(rc, "fast_topk_transform_fused")


def fast_topk_transform_ragged_fused(
    score: torch.Tensor,
    lengths: torch.Tensor,
    topk_indices_ragged: torch.Tensor,
    topk_indices_offset: torch.Tensor,
    row_starts: Optional[torch.Tensor] = None,
) -> None:
    """Top-k with a per-row offset added: ``out[i, j] = idx[i, j] + offset[i]``.

    Mirrors ``fast_topk_transform_ragged_interface``
    (``topk_indexer_radix.cu:1602-1639``).
    """
    _require(topk_indices_ragged.dim() == 2 and topk_indices_ragged.is_contiguous()
             and topk_indices_ragged.dtype == torch.int32,
             "topk_indices_ragged must be contiguous int32 2-D")
    topk = int(topk_indices_ragged.size(1))
    _check_common(score, lengths, topk, row_starts)
    B, L = score.size(0), score.size(1)
    _require(topk_indices_ragged.size(0) == B, "topk_indices_ragged.size(0) must equal B")
    _require(topk_indices_offset.dim() == 1 and topk_indices_offset.size(0) == B
             and topk_indices_offset.dtype == torch.int32 and topk_indices_offset.is_contiguous(),
             "topk_indices_offset must be contiguous int32 [B]")
    if B == 0:
        return
    lib = _lib.load()
    ws, ws_bytes = _workspace(lib, score.device, B, L, topk)
    with torch.cuda.device(score.device):
        rc = lib.ff_topk_transform_launch(
            score.data_ptr(), score.stride(0) if B > 1 else max(score.stride(0), L),
            lengths.data_ptr(), _ptr(row_starts), topk_indices_ragged.data_ptr(), B, L, topk,
            _lib.FF_EPILOGUE_ADD_OFFSET, None, 0, None, 0, topk_indices_offset.data_ptr(),
            _ptr(ws), ws_bytes, None, _stream_ptr(score.device))
    _lib.check(rc, "fast_topk_transform_ragged_fused")
