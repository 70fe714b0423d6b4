#!/usr/bin/env python
"""Benchmark of the top-k indexer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1: one step is one ``fast_topk_v3`` call on the headline configuration
(B=1, L=1,048,576, k=2048, bf16-rounded N(0,1) scores).  Inputs are resident
in HBM and rotate over 64 distinct 4 MiB rows (256 MiB > the 126 MB L2) so
every step reads cold data.  The K timed steps are replayed from one CUDA graph
and bracketed by CUDA events.
N > 1 (under torchrun): context-parallel mode, weak scaling: every rank holds a
1,048,576-column shard of one row of length N x 1,048,576; one step is ONE
kernel launch per rank (shard-local select, candidates stored into the peers
over NVLink, merge).  Time is the max over ranks.  Before anything is timed the
context-parallel result is compared, on every rank, with the one-GPU operator
on the gathered row (``parity_checked``); ``extra.c5`` adds the long-context
configuration (fp32 N(0,1), L = 4 Mi and 8 Mi split over the N ranks) beside
rank 0's one-GPU time on the same rows.

The graph of K steps is replayed until at least 50 ms of device time have
passed; ``value`` is the median per-step time over the replays and
``quantiles`` holds p20 / p50 / p80 (the reference benchmark reports the same
three, ``benchmark/bench_topk.py:374-381``).

Prints ONE JSON line (rank 0).  ``--impl reference`` times ``torch.topk`` on
the host cores for the same configuration (the CPU statement of the path); its
``reference_kernel_on_this_gpu`` says why the reference's own GPU kernel is not timed beside
it.  ``extra.reference_benchmark_rows_us`` of this library's arm is the headline shape on the
scores the reference benchmark draws for its published table.
"""
from __future__ import annotations

import argparse
import ctypes
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
# The reference has no CPU implementation of this path (its kernels are CUDA only); the CPU arm
# times the comparator the path is specified against.
CPU_IMPL_NOTE = "torch.topk on the host cores: the CPU statement of the path (the reference's own code is CUDA only)"
MIN_TIMED_MS = 50.0           # replays are repeated until this much device time has been measured


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


def measured_traffic(case: str):
    """DRAM bytes per launch of the dominant kernel from the last ncu capture of `case`, with the
    commit it was captured at (flash_float_jit_kernels_b200/measured_traffic.json), or None."""
    p = ROOT / "flash_float_jit_kernels_b200" / "measured_traffic.json"
    try:
        rec = json.loads(p.read_text())[case]
        return int(rec["dram_bytes_per_launch"]), str(rec.get("commit", "unknown"))
    except Exception:
        return None, None


def launch_shape(lib, B, L, k, hinted=False):
    """(CTAs per cluster, clusters per row) of the launch the operator makes for this shape."""
    out = (ctypes.c_int32 * 2)()
    lib.ff_topk_policy_launch_shape(B, L, k, 1, 1 if hinted else 0, out)
    return int(out[0]), int(out[1])


def quantiles(samples):
    """p20 / p50 / p80 of a list (nearest rank), as the reference benchmark reports them."""
    v = sorted(samples)
    pick = lambda q: v[min(len(v) - 1, int(q * len(v)))]
    return {"p20": round(pick(0.2), 3), "p50": round(pick(0.5), 3), "p80": round(pick(0.8), 3), "n": len(v)}


def timed_replays(graph, stream, steps_per_replay: int, min_ms: float = MIN_TIMED_MS, max_replays: int = 4000):
    """Replays `graph` back to back on `stream` until min_ms of device time have been measured
    (at least 10 replays); returns the per-step time in us of every replay (CUDA events between
    the replays, on the replay stream)."""
    per_step_us = []
    total_ms = 0.0
    while (total_ms < min_ms or len(per_step_us) < 10) and len(per_step_us) < max_replays:
        n = 10
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
        ev[0].record(stream)
        for i in range(n):
            graph.replay()
            ev[i + 1].record(stream)
        stream.synchronize()
        for i in range(n):
            ms = ev[i].elapsed_time(ev[i + 1])
            total_ms += ms
            per_step_us.append(ms * 1e3 / steps_per_replay)
    return per_step_us


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
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        samples = timed_replays(graph, side, K)
        t1 = time.perf_counter()
        clocks = sampler.summary(t0, t1)
        sampler.stop()
    q = quantiles(samples)
    us = q["p50"]
    q["mean"] = round(sum(samples) / len(samples), 3)
    peak, peak_src = measured_peak()
    algo_bytes = 4 * L
    achieved = algo_bytes / (us * 1e-6) / 1e9
    traffic, traffic_commit = measured_traffic("headline_B1_L1M_k2048")
    shape = launch_shape(lib, 1, L, k)

    # ---- end to end through the public operator with host buffers ----------
    host_in = torch.empty((1, L), dtype=torch.float32).pin_memory()
    host_in.copy_(rows[0:1].cpu())
    host_out = torch.empty((1, k), dtype=torch.int32).pin_memory()
    dev_in = torch.empty((1, L), dtype=torch.float32, device=dev)
    dev_out = torch.empty((1, k), dtype=torch.int32, device=dev)
    Ke = max(200, min(K, 1000))

    def e2e_step():
        dev_in.copy_(host_in, non_blocking=True)
        fast_topk_v3(dev_in, lengths, k, out=dev_out)
        host_out.copy_(dev_out, non_blocking=True)

    for _ in range(5):
        e2e_step()
    torch.cuda.synchronize()
    e2e_mode = "eager calls on the current stream, one CUDA event pair per step"
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(Ke + 1)]
    ev[0].record()
    for i in range(Ke):
        e2e_step()
        ev[i + 1].record()
    torch.cuda.synchronize()
    e2e_samples = [ev[i].elapsed_time(ev[i + 1]) * 1e3 for i in range(Ke)]
    e2e_q = quantiles(e2e_samples)
    e2e_us = e2e_q["p50"]
    e2e_q["mean"] = round(sum(e2e_samples) / Ke, 3)

    extra = {}
    if not args.no_extra:
        extra = bench_extras(dev, lib, peak)
        # the headline shape on the scores the reference benchmark draws for its published table
        ref_rows = reference_benchmark_rows(dev)
        extra["reference_benchmark_rows_us"] = round(_time_calls(
            lambda i: fast_topk_v3(ref_rows[i:i + 1], lengths, k, out=outs[i]), ROTATE, 4 * ROTATE, dev), 2)
        del ref_rows
        # the same steps launched in plain stream order (the default lets a select be set up while the
        # step before it still runs; each select waits for that step's completion itself)
        lib.ff_topk_set_programmatic_launch(0)
        try:
            with torch.cuda.stream(side):
                plain_graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(plain_graph, stream=side):
                    for i in range(K):
                        step(i)
                plain_graph.replay()
                side.synchronize()
                extra["headline_plain_stream_order_us"] = quantiles(timed_replays(plain_graph, side, K))["p50"]
        finally:
            lib.ff_topk_set_programmatic_launch(-1)

    cpu = cpu_baseline(rows[0:1].cpu(), k, seconds=3.0)
    line = {
        "metric": "topk_us_per_call", "value": round(us, 3), "unit": "us", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(us / 1e3, 6), "higher_is_better": False, "scaling": "weak",
        "vs_baseline": round(us / PUBLISHED_US, 4), "dtype": "f32->u32 keys", "data": "synthetic",
        "quantiles": q,
        "config": {"workload": "B=1 L=1048576 k=2048 bf16-rounded N(0,1) (heavy ties)", "B": 1, "L": L, "k": k,
                   "l2": f"inputs rotate over {ROTATE} distinct 4 MiB rows (256 MiB > 126 MB L2)",
                   "timing": f"K steps in one CUDA graph, replayed {len(samples)} times (>= {MIN_TIMED_MS:.0f} ms), CUDA "
                             "events between the replays on the replay stream; value = median per-step time; the steps are "
                             "launched with programmatic stream serialization (extra.headline_plain_stream_order_us "
                             "is the same without it)",
                   "launch_shape": {"cluster_size": int(shape[0]), "clusters_per_row": int(shape[1]),
                                    "ctas": int(shape[0]) * int(shape[1])},
                   "vs_baseline_note": "published figure is for GB300/B300 (reference README.md:52): cross-hardware"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 5), "traffic": traffic, "traffic_captured_at_commit": traffic_commit,
                     "peak_source": peak_src, "algorithmic_bytes_per_launch": algo_bytes,
                     "frac_of_nominal_8TBs": round(achieved / NOMINAL_HBM_GBS, 5)},
        "cpu_baseline": cpu,
        "e2e": {"value": round(e2e_us, 3), "unit": "us", "h2d_bytes_per_step": 4 * L, "d2h_bytes_per_step": 4 * k,
                "steps": Ke, "mode": e2e_mode, "quantiles": e2e_q},
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
                               "launch_shape": dict(zip(("cluster_size", "clusters_per_row"),
                                                        launch_shape(lib, 64, 131072, K_TOP)))}
    # the same batches as bf16 scores (half the bytes; each score is widened exactly inside the kernel)
    b16 = [(b[0].to(torch.bfloat16), b[1], b[2]) for b in batches]
    us16 = _time_calls(lambda i: fast_topk_v3(b16[i][0], b16[i][1], K_TOP, out=b16[i][2]), nb, 90, dev)
    out["b64_ragged_k2048_bf16_scores"] = {"us_per_call": round(us16, 2), "rows_per_s": round(64 / (us16 * 1e-6), 1),
                                           "algorithmic_read_bytes": int(2 * valid),
                                           "achieved_gbs": round(2 * valid / (us16 * 1e-6) / 1e9, 1)}
    del batches, b16
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
        # the decode-step form: guesses carried from step to step, and the producer handing the select
        # its survivors (every score not below the guess is listed while the scores are written)
        from flash_float_jit_kernels_b200.indexer_logits import indexer_topk, new_handover
        hint = new_threshold_hint(B, dev)
        us_hint = _time_calls(lambda i: indexer_topk(q, kc, w, l0, K_TOP, scores=sc, out=o, threshold_hint=hint), 1, 20, dev)
        hint2 = new_threshold_hint(B, dev)
        hand = new_handover(B, dev)
        status.zero_()
        step = lambda i: indexer_topk(q, kc, w, l0, K_TOP, scores=sc, out=o, threshold_hint=hint2, status=status,
                                      handover=hand)
        us_hand = _time_calls(step, 1, 20, dev)
        status.zero_()
        step(0)
        missed = int(status.item())
        o_plain = torch.empty_like(o)
        fast_topk_v3(sc, l0, K_TOP, out=o_plain)
        torch.cuda.synchronize()
        assert torch.equal(o, o_plain), "bench: the hand-over step disagrees with the plain select"
        out["indexer_logits_b64_ragged"] = {
            "producer_us": round(us_p, 2), "k_cache_bytes_read": k_bytes,
            "achieved_gbs": round(k_bytes / (us_p * 1e-6) / 1e9, 1),
            "frac_of_measured_peak": round(k_bytes / (us_p * 1e-6) / 1e9 / peak, 4),
            "producer_plus_topk_us": round(us_pt, 2),
            "producer_plus_topk_threshold_hint_us": round(us_hint, 2),
            "producer_plus_topk_hand_over_us": round(us_hand, 2),
            "hand_over_status_after_steady_state_step": missed}
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
    return {"value": round(best * 1e6, 1), "unit": "us", "cores": cores, "kind": "port",
            "implementation": CPU_IMPL_NOTE,
            "sample": f"torch.topk on the host cores, same row (B={score_cpu.shape[0]}, L={score_cpu.shape[1]}, "
                      f"k={k}), best of {n} calls in {seconds:.0f} s"}


def reference_benchmark_rows(dev) -> torch.Tensor:
    """64 rows of 1,048,576 scores as the reference benchmark draws them for its published table
    (standard normal scores normalised by their own range to [0, 1], times 255: ``benchmark/bench_topk.py:86-89``,
    ``:111-125``, ``:437``)."""
    from flash_float_jit_kernels_b200 import workloads
    return torch.cat([workloads.reference_style(1, L_SHARD, False, "gaussian", seed=42 + i, device=dev)[0]
                      for i in range(ROTATE)])


def reference_kernel_on_this_gpu():
    """The reference's own kernel, built unchanged for sm_100a, is not run: when it was (once, in a
    child process of this arm, B=1, L=1,048,576, k=2048, the reference benchmark's own scores) the
    child ended with "CUDA warning: an illegal memory access was encountered" and exit code 1.  Code
    that has faulted on a GPU of this pool is not run on it again, so the row says why it is empty."""
    return {"unavailable": "the reference's kernel (fast_topk of its TVM-FFI module, built unchanged for sm_100a) made an "
                           "illegal memory access on this pool's B200 at B=1, L=1048576, k=2048 on its own benchmark "
                           "scores; it is not run again"}


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
        "cpu_baseline": {"value": round(us, 1), "unit": "us", "cores": cores, "kind": "port",
                         "implementation": CPU_IMPL_NOTE,
                         "sample": f"{done} full-row torch.topk calls (time budget {budget_s:.0f} s)"},
        "e2e": {"value": round(us, 1), "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if N == 1 and not args.no_extra:
        line["reference_kernel_on_this_gpu"] = reference_kernel_on_this_gpu()
    print(json.dumps(line))


# ---------------------------------------------------------------------------
# ours, N > 1: context-parallel weak scaling
# ---------------------------------------------------------------------------
def _cp_graph(plan, step, K, lib, side, args, dist, dev):
    """Captures K steps into one CUDA graph when the peer-memory exchange is in use (a step is
    one kernel launch and no library call; the step counter lives in device memory).  All ranks
    replay a graph, or none does."""
    graph, launches = None, 0
    if plan.exchange == "p2p" and not args.no_graph:
        try:
            with torch.cuda.stream(side):
                before = lib.ff_topk_launch_count()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for i in range(K):
                        step(i)
                launches = lib.ff_topk_launch_count() - before
            graph = g
        except Exception:
            graph = None
    ok = torch.tensor([1 if graph is not None else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if int(ok.item()) == 0:
        graph = None
    return graph, launches


def _cp_time(plan, step, K, lib, args, dist, dev, min_ms=MIN_TIMED_MS):
    """Per-step times (us, max over ranks per replay) of the context-parallel step."""
    side = torch.cuda.Stream()
    graph, launches = _cp_graph(plan, step, K, lib, side, args, dist, dev)
    if graph is not None:
        with torch.cuda.stream(side):
            graph.replay()                                  # untimed: upload + warm-up
        side.synchronize()
    # every rank must make the same number of replays: agree on it from a first timed one
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def one_replay():
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
        return e0.elapsed_time(e1)

    first = torch.tensor([one_replay()], device=dev)
    dist.all_reduce(first, op=dist.ReduceOp.MAX)
    n_rep = int(max(10, min(400, min_ms / max(float(first.item()), 1e-3))))
    before = lib.ff_topk_launch_count()
    times = []
    for _ in range(n_rep):
        # barrier + synchronize on both sides of every timed replay; device time, max over ranks below
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        times.append(one_replay())
    dist.barrier()
    if graph is None:
        launches = (lib.ff_topk_launch_count() - before) // max(n_rep, 1)
    t = torch.tensor(times, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) * 1e3 / K for x in t.tolist()], graph is not None, int(launches)


def _cp_parity(plan, shard_of, row_ids, lengths, k, world, rank, dist, dev, hint=None):
    """Outside any timed region: for each row id, the context-parallel result of every rank is
    compared with the one-GPU operator on the gathered row (that path is checked against the CPU
    oracle by the parity tests, at these sizes too).  Returns the number of rows compared; raises
    on any mismatch on any rank."""
    from flash_float_jit_kernels_b200 import fast_topk_v3
    bad = torch.zeros(1, dtype=torch.int32, device=dev)
    n = 0
    for i in row_ids:
        shard = shard_of(i)
        got = plan(shard, lengths, shard_of.offset, threshold_hint=hint).clone()
        parts = [torch.empty_like(shard) for _ in range(world)]
        dist.all_gather(parts, shard.contiguous())
        row = torch.cat(parts, dim=1)
        want = fast_topk_v3(row, lengths, k)
        torch.cuda.synchronize()
        if rank == 0:
            check_selection(row[0], want[0], k)
        if not torch.equal(got, want):
            bad += 1
        n += 1
    dist.all_reduce(bad, op=dist.ReduceOp.SUM)
    plan.check_status()
    if int(bad.item()) != 0:
        raise SystemExit(f"bench: context-parallel result differs from the one-GPU result "
                         f"({int(bad.item())} rank-rows of {n * world})")
    return n


class _Shards:
    """Callable row id -> this rank's (1, L_local) shard, with the shard's first global column."""

    def __init__(self, shards, offset):
        self.shards, self.offset = shards, offset

    def __call__(self, i):
        return self.shards[i % self.shards.shape[0]].unsqueeze(0)


def bench_cp(args):
    import torch.distributed as dist
    from flash_float_jit_kernels_b200 import _lib, fast_topk_v3, new_threshold_hint, shard_bounds
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
    shards = _Shards(make_rows(n_rot, L_SHARD, dev, seed=1000 + rank), rank * L_SHARD)   # this rank's columns of 32 rows
    lengths = torch.tensor([L], dtype=torch.int32, device=dev)
    plan = ContextParallelTopk(1, k, dev, exchange=args.exchange)

    hint = new_threshold_hint(1, dev) if args.threshold_hint else None   # secondary measurement, not the default line

    def step(i):
        return plan(shards(i), lengths, shards.offset, threshold_hint=hint)

    for i in range(W):
        step(i)
    torch.cuda.synchronize()
    dist.barrier()
    # ---- parity on real ranks, before anything is timed: plain steps and steps with guesses ----
    rows_checked = _cp_parity(plan, shards, range(4), lengths, k, world, rank, dist, dev)
    hint_chk = new_threshold_hint(1, dev)
    rows_checked += _cp_parity(plan, shards, [0, 0, 1, 2], lengths, k, world, rank, dist, dev, hint=hint_chk)

    sampler = ClockSampler(local)
    sampler.start()
    t0 = time.perf_counter()
    samples, graphed, launches = _cp_time(plan, step, K, lib, args, dist, dev)
    t1 = time.perf_counter()
    clocks = sampler.summary(t0, t1)
    sampler.stop()
    q = quantiles(samples)
    us = q["p50"]
    q["mean"] = round(sum(samples) / len(samples), 3)
    plan.check_status()

    # ---- end to end with host shards ----------------------------------------
    host_in = torch.empty((1, L_SHARD), dtype=torch.float32).pin_memory()
    host_in.copy_(shards(0).cpu())
    host_out = torch.empty((1, k), dtype=torch.int32).pin_memory()
    dev_in = torch.empty((1, L_SHARD), dtype=torch.float32, device=dev)
    Ke = 200

    def e2e_step():
        dev_in.copy_(host_in, non_blocking=True)
        o = plan(dev_in, lengths, shards.offset)
        host_out.copy_(o, non_blocking=True)

    for _ in range(3):
        e2e_step()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(Ke):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    ems = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(ems, op=dist.ReduceOp.MAX)
    e2e_us = float(ems.item()) * 1e3 / Ke
    plan.check_status()

    # ---- the long-context configuration as stated: fp32 N(0,1), L = 4 Mi and 8 Mi over the N ranks,
    # beside one GPU (rank 0) on the same rows -----------------------------------------------------
    c5 = {}
    if not args.no_extra:
        # (16 Mi and 32 Mi are beyond the stated configuration: they show from where on sharding pays)
        for Lc in (1 << 22, 1 << 23, 1 << 24, 1 << 25):
            a, b = shard_bounds(Lc, world, rank)
            n_rows = max(4, min(64, (160 << 20) // (4 * (b - a)) + 1))      # this rank's shards exceed L2
            n_full = max(4, (160 << 20) // (4 * Lc) + 1) if rank == 0 else 0
            g = torch.Generator(device=dev)
            g.manual_seed(5000 + Lc)                                        # same rows on every rank
            full, mine = [], []
            for i in range(n_rows):
                row = torch.randn((Lc,), generator=g, device=dev, dtype=torch.float32)
                mine.append(row[a:b].clone())
                if i < n_full:
                    full.append(row)
            sh = _Shards(torch.stack(mine), a)
            len_c = torch.tensor([Lc], dtype=torch.int32, device=dev)
            for i in range(3):
                plan(sh(i), len_c, a)
            checked = _cp_parity(plan, sh, range(3), len_c, k, world, rank, dist, dev)
            rows_checked += checked
            cs, _, _ = _cp_time(plan, lambda i: plan(sh(i), len_c, a), K, lib, args, dist, dev, min_ms=20.0)
            cq = quantiles(cs)
            hint_c = new_threshold_hint(1, dev)
            for i in range(3):
                plan(sh(i), len_c, a, threshold_hint=hint_c)
            hs, _, _ = _cp_time(plan, lambda i: plan(sh(i), len_c, a, threshold_hint=hint_c), K, lib, args, dist, dev,
                                min_ms=20.0)
            us_1gpu = None
            if rank == 0:
                fullt = torch.stack(full)
                o1 = torch.empty((1, k), dtype=torch.int32, device=dev)
                us_1gpu = _time_calls(lambda i: fast_topk_v3(fullt[i:i + 1], len_c, k, out=o1), len(full), 100, dev)
                del fullt
            dist.barrier()
            if rank == 0:
                c5[str(Lc)] = {"us_1gpu": round(us_1gpu, 2), "us_cp": cq["p50"], "us_cp_quantiles": cq,
                               "speedup": round(us_1gpu / cq["p50"], 3),
                               "us_cp_threshold_hint": quantiles(hs)["p50"],
                               "shard_columns": b - a, "rows_parity_checked": checked,
                               "stated_configuration": Lc <= (1 << 23),
                               "data": "fp32 N(0,1), same seeded rows on every rank"}
            del full, mine, sh
        plan.check_status()

    if rank == 0:
        peak, peak_src = measured_peak()
        algo_bytes = 4 * L_SHARD                                    # per GPU per launch of the select kernel
        achieved = world * algo_bytes / (us * 1e-6) / 1e9           # whole job
        line = {
            "metric": "topk_us_per_call", "value": round(us, 3), "unit": "us", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": round(us / 1e3, 6), "higher_is_better": False, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32->u32 keys", "data": "synthetic",
            "quantiles": q, "parity_checked": True, "parity_rows_compared": rows_checked,
            "config": {"workload": f"context-parallel B=1 L={L} k=2048 bf16-rounded N(0,1), "
                                   f"{world} contiguous shards of {L_SHARD} columns",
                       "B": 1, "L": L, "k": k, "parallelism": f"cp{world}",
                       "threshold_hint": bool(args.threshold_hint),
                       "l2": f"each rank rotates over {n_rot} distinct 4 MiB shards (128 MiB > 126 MB L2)",
                       "timing": (f"K steps in one CUDA graph replay" if graphed else "K eager stream launches") +
                                 f", {len(samples)} replays each between barriers, CUDA events, max over ranks per "
                                 "replay, value = median per-step time",
                       "parity": "every rank's result of 8 steps (4 plain, 4 with threshold guesses) and of 3 steps "
                                 "per long-context row length equals the one-GPU operator on the gathered row",
                       "exchange": plan.describe_exchange()},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak * world, "unit": "GB/s",
                         "frac": round(achieved / (peak * world), 5), "traffic": None, "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": algo_bytes,
                         "note": "whole step (select + exchange + merge) against N x the HBM peak; no ncu capture "
                                 "of a multi-rank step is taken (ncu is never wrapped around several ranks)"},
            "e2e": {"value": round(e2e_us, 3), "unit": "us", "h2d_bytes_per_step": 4 * L_SHARD,
                    "d2h_bytes_per_step": 4 * k, "steps": Ke},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "extra": {"c5": c5},
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
