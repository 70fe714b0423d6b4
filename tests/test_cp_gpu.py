"""Context-parallel mode on GPUs: shards emulated on one device, and real ranks over NCCL when >= 2 GPUs."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("P", [1, 2, 4, 8])
@pytest.mark.parametrize("ties", [False, True])
def test_sharded_select_and_merge_on_one_device(oracle, P, ties):
    """All P shards run back to back on one GPU through the same C entry points the ranks use."""
    from flash_float_jit_kernels_b200 import _lib, shard_bounds
    lib = _lib.load()
    lib.ff_topk_set_cluster_override(0)
    dev = torch.device("cuda:0")
    B, L, k = 2, 1 << 20, 2048
    g = torch.Generator().manual_seed(100 + P)
    s = torch.randn((B, L), generator=g)
    if ties:
        s = s.to(torch.bfloat16).float()
    lengths = torch.tensor([L, L - 12345], dtype=torch.int32)
    sd, ld = s.to(dev), lengths.to(dev)
    recv = torch.empty((P, 2, B, k), dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    for r in range(P):
        a, b = shard_bounds(L, P, r)
        shard = sd[:, a:b]
        rc = lib.ff_topk_cp_local(shard.data_ptr(), shard.stride(0), ld.data_ptr(), recv[r, 1].data_ptr(),
                                  recv[r, 0].data_ptr(), B, b - a, k, a, None, 0, None, stream)
        assert rc == 0
    out = torch.empty((B, k), dtype=torch.int32, device=dev)
    rc = lib.ff_topk_cp_merge(recv[0, 0].data_ptr(), recv[0, 1].data_ptr(), P, 2 * B * k, ld.data_ptr(),
                              out.data_ptr(), B, k, None, 0, None, stream)
    assert rc == 0
    torch.cuda.synchronize()
    # the shard-local candidates themselves match the oracle's statement of step 1
    a, b = shard_bounds(L, P, P - 1)
    v, gi = oracle.cp_local(np.ascontiguousarray(s[:, a:b].numpy()), lengths.numpy(), k, a)
    assert np.array_equal(recv[P - 1, 1].cpu().numpy(), gi)
    assert np.array_equal(recv[P - 1, 0].cpu().numpy().view(np.float32), v)
    assert np.array_equal(out.cpu().numpy(), oracle.topk_c(s.numpy(), lengths.numpy(), k))


def test_short_global_rows_in_cp_mode(oracle):
    from flash_float_jit_kernels_b200 import _lib, shard_bounds
    lib = _lib.load()
    dev = torch.device("cuda:0")
    B, L, k, P = 3, 40000, 512, 4
    s = torch.randn((B, L), generator=torch.Generator().manual_seed(5))
    lengths = torch.tensor([300, 10001, 512], dtype=torch.int32)   # row 0/2: <= k; row 1 ends inside shard 1
    sd, ld = s.to(dev), lengths.to(dev)
    recv = torch.empty((P, 2, B, k), dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    for r in range(P):
        a, b = shard_bounds(L, P, r)
        shard = sd[:, a:b]
        assert lib.ff_topk_cp_local(shard.data_ptr(), shard.stride(0), ld.data_ptr(), recv[r, 1].data_ptr(),
                                    recv[r, 0].data_ptr(), B, b - a, k, a, None, 0, None, stream) == 0
    out = torch.empty((B, k), dtype=torch.int32, device=dev)
    assert lib.ff_topk_cp_merge(recv[0, 0].data_ptr(), recv[0, 1].data_ptr(), P, 2 * B * k, ld.data_ptr(),
                                out.data_ptr(), B, k, None, 0, None, stream) == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), oracle.topk_c(s.numpy(), lengths.numpy(), k))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_real_ranks_over_nccl():
    n = min(torch.cuda.device_count(), 8)
    n = 1 << (n.bit_length() - 1)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29531", str(ROOT / "tests" / "cp_rank_main.py"), "nccl"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "CP_OK" in res.stdout


# ---- peer-memory exchange (ff_topk_cp_send / ff_topk_cp_recv_merge) -------------------------
def _make_exchanges(lib, P, B, k):
    import ctypes
    exs = []
    for r in range(P):
        h = ctypes.c_void_p()
        assert lib.ff_cp_exchange_create(P, r, B, k, ctypes.byref(h)) == 0, lib.ff_last_error_string()
        exs.append(h)
    for r in range(P):                       # same process: hand the peers' base pointers over directly
        for p in range(P):
            assert lib.ff_cp_exchange_set_peer(exs[r], p, lib.ff_cp_exchange_base(exs[p])) == 0
    return exs


@pytest.mark.parametrize("P", [1, 2, 4, 8])
def test_peer_exchange_emulated_on_one_device(oracle, P):
    """All P ranks live on one GPU.  Every rank's send is enqueued before any merge, so no
    kernel ever waits for a later launch; three steps exercise both receive buffers."""
    from flash_float_jit_kernels_b200 import _lib, shard_bounds
    lib = _lib.load()
    lib.ff_topk_set_cluster_override(0)
    dev = torch.device("cuda:0")
    B, L, k = 2, 600000, 1024
    exs = _make_exchanges(lib, P, B, k)
    try:
        stream = torch.cuda.current_stream().cuda_stream
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        for step in range(3):
            s = torch.randn((B, L), generator=torch.Generator().manual_seed(300 + step)).to(torch.bfloat16).float()
            lengths = torch.tensor([L, L - 999 * step - 1], dtype=torch.int32)
            sd, ld = s.to(dev), lengths.to(dev)
            for r in range(P):
                a, b = shard_bounds(L, P, r)
                shard = sd[:, a:b]
                assert lib.ff_topk_cp_send(exs[r], shard.data_ptr(), shard.stride(0), ld.data_ptr(), b - a, a,
                                           None, 0, status.data_ptr(), stream) == 0
            outs = torch.empty((P, B, k), dtype=torch.int32, device=dev)
            for r in range(P):
                assert lib.ff_topk_cp_recv_merge(exs[r], ld.data_ptr(), outs[r].data_ptr(), status.data_ptr(),
                                                 stream) == 0
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            exp = oracle.topk_c(s.numpy(), lengths.numpy(), k)
            for r in range(P):
                assert np.array_equal(outs[r].cpu().numpy(), exp), f"step {step} rank {r}"
    finally:
        torch.cuda.synchronize()
        for h in exs:
            lib.ff_cp_exchange_destroy(h)


def test_missing_peer_ends_in_a_timeout_status_not_a_hang():
    """Rank 1 never pushes: rank 0's merge gives up after its one-second bounded wait, reports
    FF_STATUS_WAIT_TIMEOUT in the status word, and the context stays usable."""
    from flash_float_jit_kernels_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    B, L, k = 1, 50000, 256
    exs = _make_exchanges(lib, 2, B, k)
    try:
        stream = torch.cuda.current_stream().cuda_stream
        s = torch.randn((B, L), device=dev)
        lengths = torch.tensor([2 * L], dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        out = torch.empty((B, k), dtype=torch.int32, device=dev)
        assert lib.ff_topk_cp_send(exs[0], s.data_ptr(), s.stride(0), lengths.data_ptr(), L, 0, None, 0,
                                   status.data_ptr(), stream) == 0
        assert lib.ff_topk_cp_recv_merge(exs[0], lengths.data_ptr(), out.data_ptr(), status.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        assert int(status.item()) & 2, "the wait for the absent peer should have timed out"
        assert float(torch.ones(4, device=dev).sum()) == 4.0           # context still usable
    finally:
        torch.cuda.synchronize()
        for h in exs:
            lib.ff_cp_exchange_destroy(h)


def test_peer_exchange_with_shards_shorter_than_k(oracle):
    """Ragged rows: some shards hold fewer than k valid columns (or none); their runs must still
    arrive in canonical order for the sorted-run merge."""
    from flash_float_jit_kernels_b200 import _lib, shard_bounds
    lib = _lib.load()
    dev = torch.device("cuda:0")
    P, B, L, k = 4, 3, 40000, 512
    exs = _make_exchanges(lib, P, B, k)
    try:
        stream = torch.cuda.current_stream().cuda_stream
        s = torch.randn((B, L), generator=torch.Generator().manual_seed(9)).to(torch.bfloat16).float()
        lengths = torch.tensor([10100, 300, 39999], dtype=torch.int32)   # row 0 ends 100 columns into shard 1
        sd, ld = s.to(dev), lengths.to(dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        for r in range(P):
            a, b = shard_bounds(L, P, r)
            shard = sd[:, a:b]
            assert lib.ff_topk_cp_send(exs[r], shard.data_ptr(), shard.stride(0), ld.data_ptr(), b - a, a,
                                       None, 0, status.data_ptr(), stream) == 0
        out = torch.empty((B, k), dtype=torch.int32, device=dev)
        assert lib.ff_topk_cp_recv_merge(exs[2], ld.data_ptr(), out.data_ptr(), status.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert np.array_equal(out.cpu().numpy(), oracle.topk_c(s.numpy(), lengths.numpy(), k))
    finally:
        torch.cuda.synchronize()
        for h in exs:
            lib.ff_cp_exchange_destroy(h)


def test_single_kernel_step_on_one_rank(oracle):
    """world == 1: ff_topk_cp_step runs select, announcement, wait and merge as ONE launch (the
    kernel waits only for its own CTAs, all resident).  Several steps over both receive buffers,
    rows split over clusters and not, ragged and short rows, and a two-kernel step in between."""
    import ctypes
    from flash_float_jit_kernels_b200 import _lib
    from flash_float_jit_kernels_b200.topk_indexer import _ptr, _workspace
    lib = _lib.load()
    lib.ff_topk_set_cluster_override(0)
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    for (B, L, k) in ((1, 1 << 20, 2048), (3, 70000, 512)):
        h = ctypes.c_void_p()
        assert lib.ff_cp_exchange_create(1, 0, B, k, ctypes.byref(h)) == 0
        try:
            ws, ws_bytes = _workspace(lib, dev, B, L, k)
            status = torch.zeros(1, dtype=torch.int32, device=dev)
            out = torch.empty((B, k), dtype=torch.int32, device=dev)
            for step in range(5):
                s = torch.randn((B, L), generator=torch.Generator().manual_seed(700 + step)).to(torch.bfloat16).float()
                lengths = torch.full((B,), L - 17 * step, dtype=torch.int32)
                if B > 1:
                    lengths[1] = 300 + step          # <= k: identity order
                    lengths[2] = 20000 + 1000 * step
                sd, ld = s.to(dev), lengths.to(dev)
                launches = lib.ff_topk_launch_count()
                if step == 2:                        # the two-kernel form on the same exchange
                    assert lib.ff_topk_cp_send(h, sd.data_ptr(), sd.stride(0), ld.data_ptr(), L, 0, _ptr(ws),
                                               ws_bytes, status.data_ptr(), stream) == 0
                    assert lib.ff_topk_cp_recv_merge(h, ld.data_ptr(), out.data_ptr(), status.data_ptr(), stream) == 0
                    assert lib.ff_topk_launch_count() - launches == 2
                else:
                    assert lib.ff_topk_cp_step(h, sd.data_ptr(), sd.stride(0), ld.data_ptr(), out.data_ptr(), L, 0,
                                               _ptr(ws), ws_bytes, status.data_ptr(), stream) == 0
                    assert lib.ff_topk_launch_count() - launches == 1, "the step should be a single launch"
                torch.cuda.synchronize()
                assert int(status.item()) == 0
                assert np.array_equal(out.cpu().numpy(), oracle.topk_c(s.numpy(), lengths.numpy(), k)), (B, step)
        finally:
            torch.cuda.synchronize()
            lib.ff_cp_exchange_destroy(h)


def test_single_kernel_step_with_a_missing_peer_times_out():
    """Rank 1 never runs: rank 0's single-kernel step gives up after its one-second bounded wait,
    reports FF_STATUS_WAIT_TIMEOUT, and the context stays usable."""
    from flash_float_jit_kernels_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    B, L, k = 1, 50000, 256
    exs = _make_exchanges(lib, 2, B, k)
    try:
        stream = torch.cuda.current_stream().cuda_stream
        s = torch.randn((B, L), device=dev)
        lengths = torch.tensor([2 * L], dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        out = torch.empty((B, k), dtype=torch.int32, device=dev)
        launches = lib.ff_topk_launch_count()
        assert lib.ff_topk_cp_step(exs[0], s.data_ptr(), s.stride(0), lengths.data_ptr(), out.data_ptr(), L, 0,
                                   None, 0, status.data_ptr(), stream) == 0
        assert lib.ff_topk_launch_count() - launches == 1
        torch.cuda.synchronize()
        assert int(status.item()) & 2, "the wait for the absent peer should have timed out"
        assert float(torch.ones(4, device=dev).sum()) == 4.0           # context still usable
    finally:
        torch.cuda.synchronize()
        for h in exs:
            lib.ff_cp_exchange_destroy(h)


def test_plan_wrapper_surfaces_a_missing_peer_as_an_exception(oracle):
    """The Python plan passes its own status word to every step: a step whose peer never
    delivers ends by its bounded wait, and check_status() raises instead of returning stale
    indices silently.  (The peer is a second exchange on this GPU that is never stepped.)"""
    import ctypes
    from flash_float_jit_kernels_b200 import _lib
    from flash_float_jit_kernels_b200.context_parallel import ContextParallelTopk
    lib = _lib.load()
    dev = torch.device("cuda:0")
    B, L, k = 1, 50000, 256

    class TwoRankPlanWithSilentPeer(ContextParallelTopk):
        def _setup_p2p(self):
            self.world, self.rank = 2, 0
            self._both = _make_exchanges(lib, 2, B, k)
            self._ex = self._both[0]
            return True

    plan = TwoRankPlanWithSilentPeer(B, k, dev, exchange="p2p")
    try:
        s = torch.randn((B, L), device=dev)
        lengths = torch.tensor([2 * L], dtype=torch.int32, device=dev)
        plan(s, lengths, 0)
        with pytest.raises(RuntimeError, match="FF_STATUS_WAIT_TIMEOUT"):
            plan.check_status()
        assert plan.check_status() == 0, "the bits were cleared by the failed check"
        assert float(torch.ones(4, device=dev).sum()) == 4.0           # context still usable
    finally:
        torch.cuda.synchronize()
        plan._ex = None
        for h in plan._both:
            lib.ff_cp_exchange_destroy(h)


@pytest.mark.gpu
@pytest.mark.parametrize("P,L", [(2, 600000), (4, 2400000)])
def test_peer_exchange_with_threshold_guesses(oracle, P, L):
    """Every rank keeps guesses for its own shard (read and updated in place).  Consecutive steps
    score slowly drifting rows, so the guesses of the second step on hit; a wild jump makes them
    miss, which is reported and costs a histogram pass but never exactness."""
    from flash_float_jit_kernels_b200 import _lib, new_threshold_hint, shard_bounds
    from flash_float_jit_kernels_b200.topk_indexer import _ptr, _workspace
    lib = _lib.load()
    lib.ff_topk_set_cluster_override(0)
    dev = torch.device("cuda:0")
    B, k = 2, 1024
    exs = _make_exchanges(lib, P, B, k)
    try:
        stream = torch.cuda.current_stream().cuda_stream
        hints = [new_threshold_hint(B, dev) for _ in range(P)]
        base = torch.randn((B, L), generator=torch.Generator().manual_seed(41)).to(torch.bfloat16).float()
        shard_len = shard_bounds(L, P, 0)[1]
        ws, ws_bytes = _workspace(lib, dev, B, shard_len + 8, k)
        seen = []
        for step in range(5):
            drift = 0.01 * torch.randn((B, L), generator=torch.Generator().manual_seed(50 + step))
            s = (base + drift).to(torch.bfloat16).float()
            if step == 3:
                s = s * 4.0 + 10.0           # the old guesses are far too low now: too many survivors
            lengths = torch.tensor([L, L - 12345], dtype=torch.int32)
            sd, ld = s.to(dev), lengths.to(dev)
            status = torch.zeros(1, dtype=torch.int32, device=dev)
            for r in range(P):
                a, b = shard_bounds(L, P, r)
                shard = sd[:, a:b]
                assert lib.ff_topk_cp_send_hinted(exs[r], shard.data_ptr(), shard.stride(0), ld.data_ptr(), b - a, a,
                                                  hints[r].data_ptr(), hints[r].data_ptr(), _ptr(ws), ws_bytes,
                                                  status.data_ptr(), stream) == 0
            outs = torch.empty((P, B, k), dtype=torch.int32, device=dev)
            for r in range(P):
                assert lib.ff_topk_cp_recv_merge(exs[r], ld.data_ptr(), outs[r].data_ptr(), status.data_ptr(),
                                                 stream) == 0
            torch.cuda.synchronize()
            seen.append(int(status.item()))
            assert seen[-1] & ~_lib.FF_STATUS_HINT_MISSED == 0
            exp = oracle.topk_c(s.numpy(), lengths.numpy(), k)
            for r in range(P):
                assert np.array_equal(outs[r].cpu().numpy(), exp), f"step {step} rank {r}"
            for r in range(P):
                assert not torch.isnan(hints[r]).any(), "every shard is longer than k: a guess comes back"
        assert seen[0] == 0, "NaN guesses are no guesses, so nothing can miss"
        assert seen[1] == 0 and seen[2] == 0, "guesses from the previous step should hit on drifting rows"
        assert seen[3] == _lib.FF_STATUS_HINT_MISSED
    finally:
        torch.cuda.synchronize()
        for h in exs:
            lib.ff_cp_exchange_destroy(h)


@pytest.mark.gpu
def test_single_kernel_step_with_threshold_guesses(oracle):
    """world == 1, one launch per step, guesses carried from step to step; the row is split over
    clusters (1 Mi) or not (70000)."""
    import ctypes
    from flash_float_jit_kernels_b200 import _lib, new_threshold_hint
    from flash_float_jit_kernels_b200.topk_indexer import _ptr, _workspace
    lib = _lib.load()
    lib.ff_topk_set_cluster_override(0)
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    for (B, L, k) in ((1, 1 << 20, 2048), (3, 70000, 512)):
        h = ctypes.c_void_p()
        assert lib.ff_cp_exchange_create(1, 0, B, k, ctypes.byref(h)) == 0
        try:
            ws, ws_bytes = _workspace(lib, dev, B, L, k)
            hint = new_threshold_hint(B, dev)
            out = torch.empty((B, k), dtype=torch.int32, device=dev)
            base = torch.randn((B, L), generator=torch.Generator().manual_seed(900)).to(torch.bfloat16).float()
            for step in range(4):
                drift = 0.01 * torch.randn((B, L), generator=torch.Generator().manual_seed(901 + step))
                s = (base + drift).to(torch.bfloat16).float()
                lengths = torch.full((B,), L - 17 * step, dtype=torch.int32)
                sd, ld = s.to(dev), lengths.to(dev)
                status = torch.zeros(1, dtype=torch.int32, device=dev)
                launches = lib.ff_topk_launch_count()
                assert lib.ff_topk_cp_step_hinted(h, sd.data_ptr(), sd.stride(0), ld.data_ptr(), out.data_ptr(), L, 0,
                                                  hint.data_ptr(), hint.data_ptr(), _ptr(ws), ws_bytes,
                                                  status.data_ptr(), stream) == 0
                assert lib.ff_topk_launch_count() - launches == 1, "the step should be a single launch"
                torch.cuda.synchronize()
                assert int(status.item()) == 0, (B, step)
                assert np.array_equal(out.cpu().numpy(), oracle.topk_c(s.numpy(), lengths.numpy(), k)), (B, step)
        finally:
            torch.cuda.synchronize()
            lib.ff_cp_exchange_destroy(h)


# ---- several ranks in ONE launch: the single-kernel step with world > 1 on one GPU -----------
def _emulated_shape(P, B):
    """(cluster size, clusters per row) such that the CTAs of all P ranks are resident together
    (a B200 holds 15 clusters of 8 or about 36 of 4 of this kernel)."""
    if P == 2 and B == 1:
        return 8, 7
    return 4, max(2, 28 // (P * B))


def _emulated_step(lib, exs, shards, lengths_dev, outs, offsets, hints, wss, ws_bytes, status):
    import ctypes
    P = len(exs)
    vp = ctypes.c_void_p * P
    i64 = ctypes.c_int64 * P
    return lib.ff_topk_cp_step_emulated_ranks(
        P, vp(*[h.value for h in exs]), vp(*[s.data_ptr() for s in shards]), shards[0].stride(0),
        lengths_dev.data_ptr(), vp(*[o.data_ptr() for o in outs]), i64(*[s.size(1) for s in shards]), i64(*offsets),
        None if hints is None else vp(*[h.data_ptr() for h in hints]), vp(*[w.data_ptr() for w in wss]), ws_bytes,
        status.data_ptr(), torch.cuda.current_stream().cuda_stream)


def _run_emulated(oracle, P, B, L, k, make_row, steps=3, prefix=None, use_hints=False, expect_second_round=None,
                  survivor_exchange=True, expect_sx_fallback=None):
    """Plays P ranks of `steps` context-parallel steps in one launch each and compares every
    rank's result with the oracle on the unsharded rows.  Returns the status word of every step."""
    from flash_float_jit_kernels_b200 import _lib, new_threshold_hint, shard_bounds
    lib = _lib.load()
    dev = torch.device("cuda:0")
    cluster, groups = _emulated_shape(P, B)
    assert L % (4 * P) == 0, "equal shards, so that every rank gets the same launch shape"
    if prefix is not None:
        os.environ["FF_TOPK_CP_PREFIX"] = str(prefix)
    os.environ["FF_TOPK_CP_SX"] = "1" if survivor_exchange else "0"   # (the library's default is off)
    lib.ff_topk_set_cluster_override(cluster)
    lib.ff_topk_set_groups_override(groups)
    exs = _make_exchanges(lib, P, B, k)
    seen = []
    try:
        ws_bytes = int(lib.ff_topk_workspace_bytes(B, L // P, k))
        assert ws_bytes > 0
        wss = [torch.zeros(ws_bytes, dtype=torch.uint8, device=dev) for _ in range(P)]
        hints = [new_threshold_hint(B, dev) for _ in range(P)] if use_hints else None
        outs = [torch.full((B, k), -5, dtype=torch.int32, device=dev) for _ in range(P)]
        for step in range(steps):
            s, lengths = make_row(step)
            sd, ld = s.to(dev), lengths.to(dev)
            shards, offsets = [], []
            for r in range(P):
                a, b = shard_bounds(L, P, r)
                shards.append(sd[:, a:b])
                offsets.append(a)
            status = torch.zeros(1, dtype=torch.int32, device=dev)
            launches = lib.ff_topk_launch_count()
            rc = _emulated_step(lib, exs, shards, ld, outs, offsets, hints, wss, ws_bytes, status)
            assert rc == 0, lib.ff_last_error_string()
            assert lib.ff_topk_launch_count() - launches == 1
            torch.cuda.synchronize()
            bits = int(status.item())
            seen.append(bits)
            info = _lib.FF_STATUS_HINT_MISSED | _lib.FF_STATUS_CP_SECOND_ROUND | _lib.FF_STATUS_CP_SX_FALLBACK
            assert bits & ~info == 0, f"step {step}: status {bits}"
            if expect_sx_fallback is not None:
                assert bool(bits & _lib.FF_STATUS_CP_SX_FALLBACK) == expect_sx_fallback, f"step {step}: status {bits}"
            if expect_second_round is not None:
                assert bool(bits & _lib.FF_STATUS_CP_SECOND_ROUND) == expect_second_round, f"step {step}: status {bits}"
            exp = oracle.topk_c(s.numpy(), lengths.numpy(), k)
            for r in range(P):
                assert np.array_equal(outs[r].cpu().numpy(), exp), f"step {step} rank {r}"
    finally:
        torch.cuda.synchronize()
        os.environ.pop("FF_TOPK_CP_PREFIX", None)
        os.environ.pop("FF_TOPK_CP_SX", None)
        lib.ff_topk_set_cluster_override(0)
        lib.ff_topk_set_groups_override(0)
        for h in exs:
            lib.ff_cp_exchange_destroy(h)
    return seen


@pytest.mark.parametrize("P", [2, 4, 8])
@pytest.mark.parametrize("ties", [False, True])
@pytest.mark.parametrize("survivor_exchange", [False, True])
def test_single_kernel_step_with_several_ranks_in_one_launch(oracle, P, ties, survivor_exchange):
    """world > 1 in the one-launch form on i.i.d. rows.  With the exchange of survivors every rank's
    guess for the whole row fits and all ranks finish the same survivor list; without it the heads
    of the sorted runs (2k / world candidates per rank) hold the whole top-k and no second round is
    taken."""
    B, L, k = 1, 1 << 20, 2048

    def make_row(step):
        s = torch.randn((B, L), generator=torch.Generator().manual_seed(4000 + 10 * P + step))
        if ties:
            s = s.to(torch.bfloat16).float()
        return s, torch.tensor([L - 4321 * step], dtype=torch.int32)

    _run_emulated(oracle, P, B, L, k, make_row, steps=3, expect_second_round=False,
                  survivor_exchange=survivor_exchange, expect_sx_fallback=False)


@pytest.mark.parametrize("P", [2, 4, 8])
def test_survivor_exchange_with_short_and_empty_shards(oracle, P):
    """Rows that end early: the last ranks hold an empty shard, one rank a shard of a few hundred or a
    few thousand scores.  A small shard is sent whole, a middling one (too long to send, too short
    for a guess) makes every rank fall back to sorted runs; exact either way, and the next step
    works again (both receive buffers, stale regions)."""
    B, L, k = 1, 1 << 20, 1024
    shard = L // P
    tails = [0, 37, 700, 3000, 9000, shard - 5]      # scores of the row inside the rank where it ends

    def make_row(step):
        s = torch.randn((B, L), generator=torch.Generator().manual_seed(4400 + step)).to(torch.bfloat16).float()
        return s, torch.tensor([shard * (P - 1 - (step % 2) * (P > 2)) + tails[step]], dtype=torch.int32)

    _run_emulated(oracle, P, B, L, k, make_row, steps=len(tails))


def test_survivor_exchange_with_two_rows(oracle):
    P, B, L, k = 4, 2, 1 << 20, 2048

    def make_row(step):
        s = torch.randn((B, L), generator=torch.Generator().manual_seed(4500 + step))
        return s, torch.tensor([L, L - 250000 - step], dtype=torch.int32)

    _run_emulated(oracle, P, B, L, k, make_row, steps=3, expect_sx_fallback=False)


@pytest.mark.parametrize("P", [4, 8])
def test_second_round_when_the_winners_crowd_into_one_shard(oracle, P):
    """A row that rises towards its end has its whole top-k in the last shard: the heads of the
    runs are not enough, every rank sees that on the same keys, and the ranks exchange the rest."""
    B, L, k = 1, 1 << 19, 1024

    def make_row(step):
        g = torch.Generator().manual_seed(4100 + step)
        s = torch.randn((B, L), generator=g) + torch.linspace(0.0, 40.0, L).unsqueeze(0)
        if step == 1:        # equal scores everywhere: the lowest indices win, all in shard 0
            s = torch.full((B, L), 1.5)
        return s, torch.tensor([L], dtype=torch.int32)

    seen = _run_emulated(oracle, P, B, L, k, make_row, steps=4, expect_second_round=True, expect_sx_fallback=True)
    assert all(b & 16 for b in seen)


@pytest.mark.parametrize("prefix", [1, 7, 300])
def test_short_heads_fall_back_to_whole_runs(oracle, prefix):
    """Forced tiny heads (FF_TOPK_CP_PREFIX): every step needs the second round; two rows, one of
    them ending inside the second shard and one no longer than k."""
    P, B, L, k = 4, 2, 1 << 18, 512

    def make_row(step):
        s = torch.randn((B, L), generator=torch.Generator().manual_seed(4200 + step)).to(torch.bfloat16).float()
        lengths = torch.tensor([L, (L // P) + 1000 * step + 3], dtype=torch.int32)
        if step == 2:
            lengths[1] = 400      # <= k: identity order
        return s, lengths

    _run_emulated(oracle, P, B, L, k, make_row, steps=3, prefix=prefix)


def test_several_ranks_in_one_launch_with_threshold_guesses(oracle):
    P, B, L, k = 4, 1, 1 << 20, 2048
    base = torch.randn((B, L), generator=torch.Generator().manual_seed(4300)).to(torch.bfloat16).float()

    def make_row(step):
        drift = 0.01 * torch.randn((B, L), generator=torch.Generator().manual_seed(4301 + step))
        s = (base + drift).to(torch.bfloat16).float()
        if step == 3:
            s = s * 4.0 + 10.0
        return s, torch.tensor([L], dtype=torch.int32)

    seen = _run_emulated(oracle, P, B, L, k, make_row, steps=5, use_hints=True)
    assert seen[1] == 0 and seen[2] == 0, "guesses from the previous step should hit on drifting rows"
    assert seen[3] & 8, "the jump makes every shard's guess miss"
