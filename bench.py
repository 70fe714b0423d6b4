#!/usr/bin/env python
"""Benchmark of the top-k indexer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1: one step is one ``fast_topk_v3`` call on the headline configuration
(B=1, L=1,048,576, k=2048, bf16-rounded N(0,1) scores).  Inputs are resident
in HBM and rotate over 64 distinct 4 MiB rows (256 MiB > the 126 MB L2) so
every step reads cold data.  The K timed steps are replayed from one CUDA graph
and bracketed by CUDA events.
N > 1 (under torchrun): context-parallel mode, weak scaling: every rank holds a
1,048,576-column shard of one row of length N x 1,048,576; one step is local
select + NCCL all-gather of the candidates + merge.  Time is the max over
ranks.

Prints ONE JSON line (rank 0).  ``--impl reference`` times ``torch.topk`` on
the host cores for the same configuration (the CPU statement of the path).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

L_SHARD = 1 << 20
K_TOP = 2048
PUBLISHED_US = 110.7          # fast_topk_v3, B=1, L=1,048,576, k=2048 (GB300/B300), reference README.md:52
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
ROTATE = 64
# DRAM bytes per launch of the dominant kernel at the headline configuration,
# from the ncu capture summarised under profiles/ (None until captured).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 4357632   # split-row launch, profiles/topk_cluster_kernel_headline_B1_L1M_k2048.md


# ---------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------
def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Polls SM clock and clock-event reasons through NVML (read-only) in a thread."""

    def __init__(self, index: int):
        self.samples = []           # (t, sm_mhz, reasons_mask)
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self.index = index
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, mask))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self, t0: float, t1: float):
        if self.nv is None or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        nv = self.nv
        win = [s for s in self.samples if t0 <= s[0] <= t1]
        scope = "timed_region"
        if not win:
            win, scope = self.samples, "whole_run"
        mhz = sorted(s[1] for s in win)
        mask = 0
        for s in win:
            mask |= s[2]
        names = []
        for name, bit in (("hw_slowdown", nv.nvmlClocksThrottleReasonHwSlowdown),
                          ("hw_thermal_slowdown", nv.nvmlClocksThrottleReasonHwThermalSlowdown),
                          ("sw_thermal_slowdown", nv.nvmlClocksThrottleReasonSwThermalSlowdown),
                          ("sw_power_cap", nv.nvmlClocksThrottleReasonSwPowerCap),
                          ("hw_power_brake", nv.nvmlClocksThrottleReasonHwPowerBrakeSlowdown)):
            if mask & bit:
                names.append(name)
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": names,
                "samples": len(win), "scope": scope}


def make_rows(n_rows: int, L: int, device, seed: int) -> torch.Tensor:
    """bf16-rounded N(0,1) rows (heavy ties), one distinct row per rotation slot."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    x = torch.randn((n_rows, L), generator=g, device=device, dtype=torch.float32)
    return x.to(torch.bfloat16).to(torch.float32)


def check_selection(score_row: torch.Tensor, idx: torch.Tensor, k: int):
    """Cheap on-device sanity check of one result (the parity tests do the exact comparison)."""
    idx = idx.long()
    v = score_row[idx]
    assert bool((v[:-1] >= v[1:]).all()), "bench: result not in descending value order"
    thr = v[-1]
    assert int((score_row > thr).sum()) <= k - 1 < int((score_row >= thr).sum()), "bench: wrong selection"


# ---------------------------------------------------------------------------
# ours, one GPU
# ---------------------------------------------------------------------------
def bench_single(args):
    from flash_float_jit_kernels_b200 import _lib, fast_topk_v3, workloads
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    lib = _lib.load()
    K, W = args.steps, max(args.warmup, 3)
    L, k = L_SHARD, K_TOP
    rows = make_rows(ROTATE, L, dev, seed=1)
    lengths = torch.tensor([L], dtype=torch.int32, device=dev)
    outs = torch.empty((ROTATE, 1, k), dtype=torch.int32, device=dev)

    def step(i):
        fast_topk_v3(rows[i % ROTATE].unsqueeze(0), lengths, k, out=outs[i % ROTATE])

    for i in range(W):
        step(i)
    torch.cuda.synchronize()
    check_selection(rows[0], outs[0, 0], k)

    before = lib.ff_topk_launch_count()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(K):
                step(i)
        launches_per_replay = lib.ff_topk_launch_count() - before
        graph.replay()                      # untimed: graph upload + extra warm-up
        side.synchronize()
        sampler = ClockSampler(0)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e0.record(side)
        graph.replay()
        e1.record(side)
        side.synchronize()
        t1 = time.perf_counter()
        total_ms = e0.elapsed_time(e1)
        # keep the sampler running over a few more replays so short runs still get samples
        clocks = sampler.summary(t0, t1)
        if clocks.get("scope") != "timed_region":
            t0b = time.perf_counter()
            while time.perf_counter() - t0b < 0.05:
                graph.replay()
            side.synchronize()
            clocks = sampler.summary(t0b, time.perf_counter())
            clocks["scope"] = "identical_replays_after_timed_region"
        sampler.stop()
    us = total_ms * 1e3 / K
    peak, peak_src = measured_peak()
    algo_bytes = 4 * L
    achieved = algo_bytes / (us * 1e-6) / 1e9

    # ---- end to end through the public operator with host buffers ----------
    host_in = torch.empty((1, L), dtype=torch.float32).pin_memory()
    host_in.copy_(rows[0:1].cpu())
    host_out = torch.empty((1, k), dtype=torch.int32).pin_memory()
    dev_in = torch.empty((1, L), dtype=torch.float32, device=dev)
    dev_out = torch.empty((1, k), dtype=torch.int32, device=dev)
    Ke = min(K, 500)

    def e2e_step():
        dev_in.copy_(host_in, non_blocking=True)
        fast_topk_v3(dev_in, lengths, k, out=dev_out)
        host_out.copy_(dev_out, non_blocking=True)

    for _ in range(3):
        e2e_step()
    torch.cuda.synchronize()
    e2e_mode = "eager calls on the current stream"   # (one CUDA graph replay per step measured slower: 262 us)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(Ke):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    e2e_us = e0.elapsed_time(e1) * 1e3 / Ke

    extra = {}
    if not args.no_extra:
        extra = bench_extras(dev, lib, peak)

    cpu = cpu_baseline(rows[0:1].cpu(), k, seconds=3.0)
    line = {
        "metric": "topk_us_per_call", "value": round(us, 3), "unit": "us", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(us / 1e3, 6), "higher_is_better": False, "scaling": "weak",
        "vs_baseline": round(us / PUBLISHED_US, 4), "dtype": "f32->u32 keys", "data": "synthetic",
        "config": {"workload": "B=1 L=1048576 k=2048 bf16-rounded N(0,1) (heavy ties)", "B": 1, "L": L, "k": k,
                   "l2": f"inputs rotate over {ROTATE} distinct 4 MiB rows (256 MiB > 126 MB L2)",
                   "timing": "K steps in one CUDA graph replay, CUDA events on the replay stream",
                   "cluster_size": int(lib.ff_topk_policy_cluster_size(1, L, k))},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 5), "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                     "peak_source": peak_src, "algorithmic_bytes_per_launch": algo_bytes,
                     "frac_of_nominal_8TBs": round(achieved / NOMINAL_HBM_GBS, 5)},
        "cpu_baseline": cpu,
        "e2e": {"value": round(e2e_us, 3), "unit": "us", "h2d_bytes_per_step": 4 * L, "d2h_bytes_per_step": 4 * k,
                "steps": Ke, "mode": e2e_mode},
        "gpu_launches": int(launches_per_replay),
        "clocks": clocks,
        "extra": extra,
    }
    print(json.dumps(line))


def _time_calls(fn, n_variants: int, reps: int, dev):
    """CUDA-graph timing of `reps` calls cycling over n_variants inputs; returns us per call."""
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for i in range(min(3, n_variants)):
            fn(i)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(reps):
                fn(i % n_variants)
        graph.replay()
        side.synchronize()
        best = None
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            graph.replay()
            e1.record(side)
            side.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
    return best * 1e3 / reps


def bench_extras(dev, lib, peak):
    """Secondary configurations: ragged B=64 decode batch (rows/s), latency sweep, small k."""
    from flash_float_jit_kernels_b200 import fast_topk_v3, workloads
    out = {}
    # ragged decode batch, B=64, stride 131072; 9 distinct batches = 302 MB > L2
    nb = 9
    batches = []
    for j in range(nb):
        s, l, _ = workloads.lightning_indexer_logits(64, 131072, 4096, seed=2 + j, device=dev)
        batches.append((s, l, torch.empty((64, K_TOP), dtype=torch.int32, device=dev)))
    us = _time_calls(lambda i: fast_topk_v3(batches[i][0], batches[i][1], K_TOP, out=batches[i][2]), nb, 90, dev)
    valid = sum(int(b[1].sum()) for b in batches) / nb
    gbs = 4 * valid / (us * 1e-6) / 1e9
    out["b64_ragged_k2048"] = {"us_per_call": round(us, 2), "rows_per_s": round(64 / (us * 1e-6), 1),
                               "algorithmic_read_bytes": int(4 * valid), "achieved_gbs": round(gbs, 1),
                               "frac_of_measured_peak": round(gbs / peak, 4),
                               "frac_of_nominal_8TBs": round(gbs / NOMINAL_HBM_GBS, 4),
                               "cluster_size": int(lib.ff_topk_policy_cluster_size(64, 131072, K_TOP))}
    del batches
    sweep = {}
    for L in (16384, 65536, 131072, 262144, 524288):
        n = max(2, min(64, (300 << 20) // (4 * L)))
        rows = make_rows(n, L, dev, seed=10)
        lengths = torch.tensor([L], dtype=torch.int32, device=dev)
        o = torch.empty((1, K_TOP), dtype=torch.int32, device=dev)
        sweep[str(L)] = round(_time_calls(lambda i: fast_topk_v3(rows[i:i + 1], lengths, K_TOP, out=o), n, 400, dev), 2)
    out["latency_sweep_us_B1_k2048"] = sweep
    small = {}
    for B in (1, 4):
        for k in (512, 1024):
            n = 16 if B == 4 else 64
            s, l, _ = workloads.gaussian_outliers(B * n, L_SHARD, seed=3, device=dev)
            s = s.view(n, B, L_SHARD)
            lengths = torch.full((B,), L_SHARD, dtype=torch.int32, device=dev)
            o = torch.empty((B, k), dtype=torch.int32, device=dev)
            small[f"B{B}_k{k}"] = round(_time_calls(lambda i: fast_topk_v3(s[i], lengths, k, out=o), n, 200, dev), 2)
            del s
    out["outlier_tail_us_L1M"] = small
    # Threshold guesses carried from call to call (fast_topk_v3(threshold_hint=...)): the decode-stream
    # use, where consecutive calls see similar rows.  Same inputs as above (the headline's 64 rotating
    # rows; one ragged batch whose rows are perturbed from step to step), exact results either way.
    from flash_float_jit_kernels_b200 import new_threshold_hint
    hinted = {}
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def missed_steps(call, n, steps=24):
        miss = 0
        for i in range(steps):
            status.zero_()
            call(i % n)
            miss += int(status.item()) != 0
        return miss

    rows = make_rows(64, L_SHARD, dev, seed=1)
    lengths = torch.tensor([L_SHARD], dtype=torch.int32, device=dev)
    o = torch.empty((1, K_TOP), dtype=torch.int32, device=dev)
    hint = new_threshold_hint(1, dev)
    call = lambda i: fast_topk_v3(rows[i:i + 1], lengths, K_TOP, out=o, status=status, threshold_hint=hint)
    hinted["B1_L1M_us"] = round(_time_calls(call, 64, 400, dev), 2)
    hinted["B1_L1M_missed_steps_of_24"] = missed_steps(call, 64)
    del rows
    s0, l0, _ = workloads.lightning_indexer_logits(64, 131072, 4096, seed=2, device=dev)
    g = torch.Generator(device=dev)
    g.manual_seed(77)
    steps = [s0 + 0.02 * j * torch.randn(s0.shape, generator=g, device=dev) for j in range(9)]   # 302 MB > L2
    o = torch.empty((64, K_TOP), dtype=torch.int32, device=dev)
    hint = new_threshold_hint(64, dev)
    plain = lambda i: fast_topk_v3(steps[i], l0, K_TOP, out=o)
    call = lambda i: fast_topk_v3(steps[i], l0, K_TOP, out=o, status=status, threshold_hint=hint)
    hinted["b64_ragged_plain_us"] = round(_time_calls(plain, 9, 90, dev), 2)
    hinted["b64_ragged_us"] = round(_time_calls(call, 9, 90, dev), 2)
    hinted["b64_ragged_rows_per_s"] = round(64 / (hinted["b64_ragged_us"] * 1e-6), 1)
    hinted["b64_ragged_missed_steps_of_24"] = missed_steps(call, 9)
    out["threshold_hint"] = hinted
    del steps, s0
    # The step before the path: the indexer-logit producer (tcgen05 kernel) on the same ragged
    # batch shape, from an fp8 K cache of 64 x 131072 keys (1 GiB, far larger than L2), alone and
    # followed by the top-k.  Bound: the K bytes read once from HBM.
    try:
        from flash_float_jit_kernels_b200.indexer_logits import indexer_logits_fp8
        g = torch.Generator(device=dev)
        g.manual_seed(5)
        B, Lm = 64, 131072
        f8 = torch.float8_e4m3fn
        q = (torch.randn((B, 64, 128), generator=g, device=dev) / 4).to(f8)
        w = torch.rand((B, 64), generator=g, device=dev)
        kc = torch.empty((B, Lm, 128), dtype=f8, device=dev)
        for b in range(B):
            kc[b] = (torch.randn((Lm, 128), generator=g, device=dev) / 4).to(f8)
        sc = torch.full((B, Lm), float("-inf"), device=dev)
        o = torch.empty((B, K_TOP), dtype=torch.int32, device=dev)
        k_bytes = 128 * int(l0.sum())
        us_p = _time_calls(lambda i: indexer_logits_fp8(q, kc, w, l0, out=sc), 1, 20, dev)
        us_pt = _time_calls(lambda i: (indexer_logits_fp8(q, kc, w, l0, out=sc), fast_topk_v3(sc, l0, K_TOP, out=o)), 1, 20, dev)
        out["indexer_logits_b64_ragged"] = {
            "producer_us": round(us_p, 2), "k_cache_bytes_read": k_bytes,
            "achieved_gbs": round(k_bytes / (us_p * 1e-6) / 1e9, 1),
            "frac_of_measured_peak": round(k_bytes / (us_p * 1e-6) / 1e9 / peak, 4),
            "producer_plus_topk_us": round(us_pt, 2)}
        del kc, sc
    except Exception as e:   # the producer is a separate library; its absence must not hide the top-k numbers
        out["indexer_logits_b64_ragged"] = {"error": str(e)[:200]}
    return out


# ---------------------------------------------------------------------------
# CPU baseline / reference arm: torch.topk on the host cores
# ---------------------------------------------------------------------------
def cpu_baseline(score_cpu: torch.Tensor, k: int, seconds: float):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    t_end = time.perf_counter() + seconds
    best, n = None, 0
    torch.topk(score_cpu, k, dim=-1)
    while time.perf_counter() < t_end or n < 3:
        t0 = time.perf_counter()
        torch.topk(score_cpu, k, dim=-1)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
        n += 1
    return {"value": round(best * 1e6, 1), "unit": "us", "cores": cores, "kind": "reference",
            "sample": f"torch.topk on the host cores, same row (B={score_cpu.shape[0]}, L={score_cpu.shape[1]}, "
                      f"k={k}), best of {n} calls in {seconds:.0f} s"}


def bench_reference(args):
    """The CPU statement of the path (torch.topk, all host threads) on the same configuration."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    N = args.gpus
    K, W = args.steps, max(args.warmup, 3)
    L = L_SHARD * N
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    rows = make_rows(4, L, "cpu", seed=1)
    budget_s = 120.0
    for i in range(W):
        torch.topk(rows[i % 4:i % 4 + 1], K_TOP, dim=-1)
    t0 = time.perf_counter()
    done = 0
    for i in range(K):
        torch.topk(rows[i % 4:i % 4 + 1], K_TOP, dim=-1)
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    us = (time.perf_counter() - t0) * 1e6 / done
    line = {
        "impl": "reference", "metric": "topk_us_per_call", "value": round(us, 1), "unit": "us", "n_gpus": N,
        "steps": done, "warmup": W, "ms_per_step": round(us / 1e3, 4), "higher_is_better": False,
        "scaling": "weak", "vs_baseline": round(us / PUBLISHED_US, 3), "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"B=1 L={L} k=2048 bf16-rounded N(0,1) (heavy ties), torch.topk on host cores",
                   "B": 1, "L": L, "k": K_TOP},
        "cpu_baseline": {"value": round(us, 1), "unit": "us", "cores": cores, "kind": "reference",
                         "sample": f"{done} full-row torch.topk calls (time budget {budget_s:.0f} s)"},
        "e2e": {"value": round(us, 1), "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------
# ours, N > 1: context-parallel weak scaling
# ---------------------------------------------------------------------------
def bench_cp(args):
    import torch.distributed as dist
    from flash_float_jit_kernels_b200 import _lib
    from flash_float_jit_kernels_b200.context_parallel import ContextParallelTopk
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    lib = _lib.load()
    K, W = args.steps, max(args.warmup, 3)
    L, k = L_SHARD * world, K_TOP
    n_rot = 32
    shards = make_rows(n_rot, L_SHARD, dev, seed=1000 + rank)       # this rank's columns of 32 distinct rows
    lengths = torch.tensor([L], dtype=torch.int32, device=dev)
    plan = ContextParallelTopk(1, k, dev, exchange=args.exchange)
    offset = rank * L_SHARD

    hint = None
    if args.threshold_hint:                                          # secondary measurement, not the default line
        from flash_float_jit_kernels_b200 import new_threshold_hint
        hint = new_threshold_hint(1, dev)

    def step(i):
        return plan(shards[i % n_rot].unsqueeze(0), lengths, offset, threshold_hint=hint)

    for i in range(W):
        step(i)
    torch.cuda.synchronize()
    dist.barrier()
    # With the peer-memory exchange a step is one kernel launch and no library call, so the
    # K steps are captured into one CUDA graph (the step counter lives in device memory);
    # with the NCCL exchange they are launched eagerly.
    graph = None
    side = torch.cuda.Stream()
    if plan.exchange == "p2p" and not args.no_graph:
        try:
            with torch.cuda.stream(side):
                before_cap = lib.ff_topk_launch_count()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for i in range(K):
                        step(i)
                launches_per_replay = lib.ff_topk_launch_count() - before_cap
            graph = g
        except Exception:
            graph = None
    ok = torch.tensor([1 if graph is not None else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)           # all ranks replay a graph, or none does
    if int(ok.item()) == 0:
        graph = None
    if graph is not None:
        with torch.cuda.stream(side):
            graph.replay()                                  # untimed: upload + warm-up
        side.synchronize()
    before = lib.ff_topk_launch_count()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    if graph is not None:
        with torch.cuda.stream(side):
            e0.record(side)
            graph.replay()
            e1.record(side)
        side.synchronize()
    else:
        e0.record()
        for i in range(K):
            step(i)
        e1.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    dist.barrier()
    launches = launches_per_replay if graph is not None else lib.ff_topk_launch_count() - before
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    clocks = sampler.summary(t0, t1)
    sampler.stop()
    us = float(ms.item()) * 1e3 / K

    # end to end with host shards
    host_in = torch.empty((1, L_SHARD), dtype=torch.float32).pin_memory()
    host_in.copy_(shards[0:1].cpu())
    host_out = torch.empty((1, k), dtype=torch.int32).pin_memory()
    dev_in = torch.empty((1, L_SHARD), dtype=torch.float32, device=dev)
    Ke = min(K, 200)

    def e2e_step():
        dev_in.copy_(host_in, non_blocking=True)
        o = plan(dev_in, lengths, offset)
        host_out.copy_(o, non_blocking=True)

    for _ in range(3):
        e2e_step()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(Ke):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    ems = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(ems, op=dist.ReduceOp.MAX)
    e2e_us = float(ems.item()) * 1e3 / Ke

    if rank == 0:
        peak, peak_src = measured_peak()
        algo_bytes = 4 * L_SHARD                                    # per GPU per launch of the select kernel
        achieved = world * algo_bytes / (us * 1e-6) / 1e9           # whole job
        line = {
            "metric": "topk_us_per_call", "value": round(us, 3), "unit": "us", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": round(us / 1e3, 6), "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32->u32 keys", "data": "synthetic",
            "config": {"workload": f"context-parallel B=1 L={L} k=2048 bf16-rounded N(0,1), "
                                   f"{world} contiguous shards of {L_SHARD} columns",
                       "B": 1, "L": L, "k": k, "parallelism": f"cp{world}",
                       "threshold_hint": bool(args.threshold_hint),
                       "l2": f"each rank rotates over {n_rot} distinct 4 MiB shards (128 MiB > 126 MB L2)",
                       "timing": ("K steps in one CUDA graph replay" if graph is not None else
                                  "eager stream launches") + ", CUDA events, max over ranks",
                       "exchange": ("self-validating 16-byte entries stored into every peer's receive buffer "
                                    "over NVLink from the select kernel (32 KiB per rank per peer); the same "
                                    "launch polls its local entries and merges" if plan.exchange == "p2p" else
                                    "NCCL all-gather of (value, global index) candidates, 16 KiB per rank")},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak * world, "unit": "GB/s",
                         "frac": round(achieved / (peak * world), 5), "traffic": None, "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": algo_bytes,
                         "note": "whole step (select + exchange + merge) against N x the HBM peak"},
            "e2e": {"value": round(e2e_us, 3), "unit": "us", "h2d_bytes_per_step": 4 * L_SHARD,
                    "d2h_bytes_per_step": 4 * k, "steps": Ke},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        print(json.dumps(line))
    plan.close()
    dist.destroy_process_group()


def run_profile_case(args):
    """A handful of eager launches of one configuration, for ncu captures (prints no bench value)."""
    from flash_float_jit_kernels_b200 import fast_topk_v3, workloads
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    name = args.profile_case
    if name == "logits":
        # the indexer-logit producer on a ragged batch of 32 rows x 65,536 keys (256 MiB of fp8 K, larger than L2)
        from flash_float_jit_kernels_b200.indexer_logits import indexer_logits_fp8
        g = torch.Generator(device=dev)
        g.manual_seed(5)
        B, Lm = 32, 65536
        f8 = torch.float8_e4m3fn
        q = (torch.randn((B, 64, 128), generator=g, device=dev) / 4).to(f8)
        w = torch.rand((B, 64), generator=g, device=dev)
        kc = torch.empty((B, Lm, 128), dtype=f8, device=dev)
        for b in range(B):
            kc[b] = (torch.randn((Lm, 128), generator=g, device=dev) / 4).to(f8)
        lens = torch.randint(4096, Lm + 1, (B,), generator=g, device=dev, dtype=torch.int32)
        sc = torch.full((B, Lm), float("-inf"), device=dev)
        for _ in range(max(args.warmup, 1) + args.steps):
            indexer_logits_fp8(q, kc, w, lens, out=sc)
        torch.cuda.synchronize()
        print(json.dumps({"profile_case": name, "launches": max(args.warmup, 1) + args.steps,
                          "k_bytes_per_launch": 128 * int(lens.sum())}))
        return
    n_rot = 40   # 40 x 4 MiB = 160 MiB > L2 for the 1M-column cases
    if name == "headline":
        rows = make_rows(n_rot, L_SHARD, dev, seed=1).view(n_rot, 1, L_SHARD)
        lengths = torch.tensor([L_SHARD], dtype=torch.int32, device=dev)
        k = K_TOP
    elif name == "unique16k":
        n_rot = 8
        rows = torch.stack([workloads.gaussian_unique(1, 16384, seed=i, device=dev)[0] for i in range(n_rot)])
        lengths = torch.tensor([16384], dtype=torch.int32, device=dev)
        k = K_TOP
    elif name == "b64":
        n_rot = 5
        batches = [workloads.lightning_indexer_logits(64, 131072, 4096, seed=2 + j, device=dev) for j in range(n_rot)]
        rows = torch.stack([b[0] for b in batches])
        lens = [b[1] for b in batches]
        k = K_TOP
    else:
        raise SystemExit(f"unknown profile case {name}")
    out = torch.empty((rows.shape[1], k), dtype=torch.int32, device=dev)
    for i in range(max(args.warmup, 1) + args.steps):
        l = lens[i % n_rot] if name == "b64" else lengths
        fast_topk_v3(rows[i % n_rot], l, k, out=out)
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": name, "launches": max(args.warmup, 1) + args.steps}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary configurations")
    ap.add_argument("--no-graph", action="store_true", help="N > 1: launch the steps eagerly instead of replaying a graph")
    ap.add_argument("--threshold-hint", action="store_true",
                    help="N > 1: every rank carries a threshold guess for its shard from step to step")
    ap.add_argument("--exchange", default="auto", choices=["auto", "p2p", "nccl"], help="N > 1: candidate exchange")
    ap.add_argument("--profile-case", default=None, choices=["headline", "unique16k", "b64", "logits"],
                    help="run a few eager launches of one configuration and exit (for ncu)")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args)
        return
    if args.impl == "reference":
        bench_reference(args)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        bench_cp(args)
    else:
        if args.gpus > 1:
            raise SystemExit("launch N > 1 with torch.distributed.run (one rank per GPU)")
        bench_single(args)


if __name__ == "__main__":
    main()
