"""Context-parallel top-k: the L axis of every row is sharded over the ranks.

The reference has no multi-GPU mode (its "distributed" means CTAs of one
thread-block cluster, ``topk_indexer_radix.cu:554-973``); the semantics here
are those of ``fast_topk_v3`` (``jit_kernel/topk_indexer.py:109``) applied to
the unsharded row.

Three steps per call, all on the current stream:
  1. local select on the shard -> ``k`` candidates ``(value, global index)``
     per row, in canonical order;
  2. exchange of the candidate blocks (``2*B*k*4`` bytes per rank);
  3. exact merge-select of the ``P*k`` candidates.

Two exchanges are implemented.  ``p2p`` (default on GPUs): every rank stores its
candidates straight into every peer's receive buffer over NVLink (peer memory
mapped through CUDA IPC) as self-validating 16-byte entries ``{value, step, index, step}``,
and the same kernel then polls its own (local) entries with a bounded wait and
merges -- one kernel launch per step, no fence, no flag, no collective library
call (``ff_topk_cp_step``).  ``nccl``: ``all_gather_into_tensor`` between
``ff_topk_cp_local`` and ``ff_topk_cp_merge``; kept as the baseline and as the
fallback when peer memory cannot be mapped.

Exactness: shards are contiguous, so the order (value desc, global index asc)
restricted to one shard equals that shard's local order; every global winner
is among its shard's local top-k; merging under the same total order is exact.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib
from .topk_indexer import TopkArgumentError, _check_common, _ptr, _require, _stream_ptr, _workspace


def shard_bounds(L: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Columns ``[start, end)`` of rank ``rank``: equal contiguous pieces of
    ``L // world_size`` columns (rounded down to a multiple of 4 so every shard
    starts 16-byte aligned); the last rank takes the remainder."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise TopkArgumentError(f"bad rank {rank} for world size {world_size}")
    base = (L // world_size) & ~3
    if base == 0:
        base = L // world_size
    start = rank * base
    end = L if rank == world_size - 1 else start + base
    return start, end


class ContextParallelTopk:
    """Reusable context-parallel top-k for one (B, k) shape.

    Keeps the candidate send/receive buffers so that repeated calls allocate
    nothing.  ``group`` is a ``torch.distributed`` process group (NCCL on GPUs).
    """

    def __init__(self, B: int, topk: int, device: torch.device, group=None, exchange: str = "auto"):
        _require(1 <= topk <= _lib.FF_TOPK_MAX_K, f"topk must be in [1, {_lib.FF_TOPK_MAX_K}]")
        _require(exchange in ("auto", "p2p", "nccl"), "exchange must be 'auto', 'p2p' or 'nccl'")
        self.B = B
        self.k = topk
        self.device = torch.device(device)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._ex = None
        self.exchange = "nccl"
        if exchange != "nccl" and self.device.type == "cuda":
            if self._setup_p2p():
                self.exchange = "p2p"
            elif exchange == "p2p":
                raise RuntimeError("peer-memory exchange could not be set up on every rank")
        # Soft-error bits of every step accumulate here (the kernels OR into it); see check_status().
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # plane 0: value bits, plane 1: global index
        self.send = torch.empty((2, B, topk), dtype=torch.int32, device=self.device)
        self.recv = torch.empty((self.world, 2, B, topk), dtype=torch.int32, device=self.device)
        self.out = torch.empty((B, topk), dtype=torch.int32, device=self.device)

    # -- peer-memory exchange ---------------------------------------------
    def _setup_p2p(self) -> bool:
        """Allocates this rank's exchange buffers and maps every peer's (CUDA IPC).
        All ranks agree on the outcome; on any failure everything is released."""
        lib = _lib.load()
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            ok = lib.ff_cp_exchange_create(self.world, self.rank, self.B, self.k, ctypes.byref(handle)) == 0
            blob = ctypes.create_string_buffer(64)
            if ok and self.world > 1:
                ok = lib.ff_cp_exchange_ipc_handle(handle, blob) == 0
            if self.world > 1:
                gathered = [None] * self.world
                dist.all_gather_object(gathered, (ok, blob.raw), group=self.group)
                ok = all(g[0] for g in gathered)
                if ok:
                    handles = b"".join(g[1] for g in gathered)
                    ok = lib.ff_cp_exchange_open_peers(handle, handles, self.world) == 0
                gathered = [None] * self.world
                dist.all_gather_object(gathered, ok, group=self.group)
                ok = all(gathered)
            if not ok:
                if handle.value:
                    lib.ff_cp_exchange_destroy(handle)
                return False
        self._ex = handle
        return True

    def close(self) -> None:
        """Releases the peer mappings and buffers (collective: every rank calls it, so that no
        rank unmaps a buffer a peer's kernel may still store into)."""
        if self._ex is not None:
            torch.cuda.synchronize(self.device)
            if self.world > 1 and dist.is_initialized():
                dist.barrier(group=self.group)
            self._release()

    def _release(self) -> None:
        """Non-collective release of this rank's exchange allocation and peer mappings."""
        ex, self._ex = self._ex, None
        if ex is not None:
            try:
                _lib.load().ff_cp_exchange_destroy(ex)
            except Exception:     # interpreter shutdown: the driver reclaims the memory with the process
                pass

    def __enter__(self) -> "ContextParallelTopk":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def __del__(self):
        # A plan that was never closed must not leak its allocation.  No barrier is possible in a
        # finalizer, so only this rank's side is released, after its own work has drained; peers
        # that are still stepping would fault, which is why close() is the documented way out.
        if getattr(self, "_ex", None) is not None:
            try:
                torch.cuda.synchronize(self.device)
            except Exception:
                pass
            self._release()

    def describe_exchange(self) -> str:
        """One line saying how candidates travel between the ranks (for benchmark records)."""
        if self.exchange == "p2p":
            return ("self-validating 16-byte entries stored into every peer's receive buffer over NVLink from "
                    "the select kernel; the same launch polls its local entries and merges")
        return "NCCL all-gather of (value, global index) candidates, 16 KiB per rank"

    def check_status(self, reset: bool = True) -> int:
        """Reads the accumulated soft-error bits (this synchronises the device, so call it at a
        point of your choosing, not per step).  ``FF_STATUS_WAIT_TIMEOUT`` (2) means a peer's
        entries did not arrive within the bounded wait: the affected step's result is INVALID
        (slots it could not fill keep older contents) and the ranks may be more than one step
        apart, which the two alternating receive buffers do not cover.  Before stepping again,
        re-synchronise every rank (a host barrier with all streams drained) or build a new plan.
        Raises ``RuntimeError`` on that bit; returns the other bits (information only)."""
        bits = int(self.status.item())
        if reset and bits:
            self.status.zero_()
        if bits & _lib.FF_STATUS_WAIT_TIMEOUT:
            raise RuntimeError(
                "context-parallel top-k: a bounded wait ran out (FF_STATUS_WAIT_TIMEOUT): a result since the "
                "last check is invalid; re-synchronise all ranks (barrier) or re-create the plan before the next step")
        return bits

    def _step_p2p(self, score_shard: torch.Tensor, lengths: torch.Tensor, shard_offset: int,
                  threshold_hint: Optional[torch.Tensor] = None) -> None:
        lib = _lib.load()
        B, L = score_shard.size(0), score_shard.size(1)
        ws, ws_bytes = _workspace(lib, score_shard.device, B, L, self.k)
        hint = threshold_hint.data_ptr() if threshold_hint is not None else None
        with torch.cuda.device(score_shard.device):
            rc = lib.ff_topk_cp_step_hinted(
                self._ex, score_shard.data_ptr(), score_shard.stride(0) if B > 1 else max(score_shard.stride(0), L),
                lengths.data_ptr(), self.out.data_ptr(), L, shard_offset, hint, hint, _ptr(ws), ws_bytes,
                self.status.data_ptr(), _stream_ptr(score_shard.device))
        _lib.check(rc, "ff_topk_cp_step_hinted")

    # -- step 1 ---------------------------------------------------------
    def _local(self, score_shard: torch.Tensor, lengths: torch.Tensor, shard_offset: int) -> None:
        lib = _lib.load()
        B, L = score_shard.size(0), score_shard.size(1)
        ws, ws_bytes = _workspace(lib, score_shard.device, B, L, self.k)
        with torch.cuda.device(score_shard.device):
            rc = lib.ff_topk_cp_local(
                score_shard.data_ptr(), score_shard.stride(0) if B > 1 else max(score_shard.stride(0), L),
                lengths.data_ptr(), self.send[1].data_ptr(), self.send[0].data_ptr(),
                B, L, self.k, shard_offset, _ptr(ws), ws_bytes, self.status.data_ptr(),
                _stream_ptr(score_shard.device))
        _lib.check(rc, "ff_topk_cp_local")

    # -- step 2 ---------------------------------------------------------
    def _exchange(self) -> None:
        if self.world == 1:
            self.recv[0].copy_(self.send)
        else:
            dist.all_gather_into_tensor(self.recv.view(-1), self.send.view(-1), group=self.group)

    # -- step 3 ---------------------------------------------------------
    def _merge(self, lengths: torch.Tensor) -> None:
        lib = _lib.load()
        n_cand = self.world * self.k
        ws, ws_bytes = _workspace(lib, self.device, self.B, n_cand, self.k)
        with torch.cuda.device(self.device):
            rc = lib.ff_topk_cp_merge(
                self.recv[0, 0].data_ptr(), self.recv[0, 1].data_ptr(), self.world,
                2 * self.B * self.k, lengths.data_ptr(), self.out.data_ptr(), self.B, self.k,
                _ptr(ws), ws_bytes, self.status.data_ptr(), _stream_ptr(self.device))
        _lib.check(rc, "ff_topk_cp_merge")

    def __call__(self, score_shard: torch.Tensor, lengths: torch.Tensor, shard_offset: int,
                 threshold_hint: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``score_shard``: (B, L_local) columns ``[shard_offset, shard_offset+L_local)``
        of the full rows; ``lengths``: (B) int32 GLOBAL row lengths (identical on
        every rank).  Returns (B, k) int32 global indices, identical on every rank.

        ``threshold_hint``: optional (B) float32 tensor of THIS rank
        (:func:`new_threshold_hint`), read and updated: guesses for the shard-local
        select, with the meaning of ``fast_topk_v3(threshold_hint=...)``.  Used by the
        peer-memory exchange only; the result is exact with or without it."""
        if threshold_hint is not None:
            _require(threshold_hint.shape == (self.B,) and threshold_hint.dtype == torch.float32
                     and threshold_hint.is_contiguous() and threshold_hint.device == score_shard.device,
                     "threshold_hint must be a contiguous (B) float32 tensor on score_shard's device")
        _require(score_shard.dim() == 2 and score_shard.size(0) == self.B, "score_shard must be [B, L_local]")
        _require(lengths.dim() == 1 and lengths.size(0) == self.B and lengths.dtype == torch.int32
                 and lengths.is_contiguous(), "lengths must be contiguous int32 [B]")
        _require(shard_offset >= 0, "shard_offset must be >= 0")
        if self._ex is not None:
            self._step_p2p(score_shard, lengths, int(shard_offset), threshold_hint)
            return self.out
        self._local(score_shard, lengths, int(shard_offset))
        self._exchange()
        self._merge(lengths)
        return self.out


_PLANS: dict = {}


def fast_topk_v3_cp(
    score_shard: torch.Tensor,
    lengths: torch.Tensor,
    topk: int,
    shard_offset: int,
    group=None,
    plan: Optional[ContextParallelTopk] = None,
) -> torch.Tensor:
    """Functional form of :class:`ContextParallelTopk`.  Without ``plan`` the plan for this
    (device, group, B, topk) is built on first use (a collective: every rank must make the same
    first call) and kept for later calls, so a per-step call allocates nothing; release the kept
    plans with :func:`close_cached_plans`."""
    _check_common(score_shard, lengths, topk, None)
    if plan is None:
        key = (score_shard.device, id(group) if group is not None else None, score_shard.size(0), topk)
        plan = _PLANS.get(key)
        if plan is None:
            plan = ContextParallelTopk(score_shard.size(0), topk, score_shard.device, group)
            _PLANS[key] = plan
    return plan(score_shard, lengths, shard_offset)


def close_cached_plans() -> None:
    """Closes the plans :func:`fast_topk_v3_cp` keeps (collective, like ``ContextParallelTopk.close``)."""
    while _PLANS:
        _, plan = _PLANS.popitem()
        plan.close()
