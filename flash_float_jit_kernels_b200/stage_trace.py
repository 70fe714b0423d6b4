"""Per-CTA stage timeline of one top-k launch.

    python -m flash_float_jit_kernels_b200.stage_trace [--case NAME] [--cluster C]

Switches on the library's trace buffer (``ff_topk_set_trace_buffer``), runs one
launch after a few warm-up launches, and prints for the first and last CTA how
long each stage of the kernel took (SM cycle counter, converted with the SM
clock reported by the driver).  It plays the role of the reference's
``SMALL_K_PROFILE`` clock64 brackets (``top_small_k.cuh:39-41,132-135``) and of
its exported stage timeline (``benchmark/viz/topk``).
"""
from __future__ import annotations

import argparse

import torch

from . import _lib, fast_topk_v3, workloads

# slot -> name, in execution order (slots as written by FF_TRACE in csrc/ff_topk_kernel.cuh)
STAGES = [
    (0, "start"), (21, "own_guess"), (1, "sweep1_hist"), (26, "merge_barrier"), (27, "merge_remote_loads"),
    (28, "merge_scan"), (29, "merge_fine_loads"), (30, "merge_threshold"), (2, "merge_end"),
    (3, "sweep2_collect"), (4, "gather_to_peers"), (38, "survivor_regions_read"), (39, "survivor_list_loaded"), (20, "final_barrier"), (22, "finish_bin_hist"),
    (23, "finish_scan"), (24, "finish_scatter"), (31, "finish_rank_in_buckets"), (25, "finish_rank_emit"),
    # context-parallel single-kernel step only
    (32, "select_done"), (36, "merge_start"), (33, "peer_heads_staged"), (37, "own_candidate_ranked"), (34, "heads_checked"),
    (35, "merged_and_written"),
]

def _gaussian_row(L, dev):
    g = torch.Generator(device=dev)
    g.manual_seed(3)
    return (torch.randn((1, L), generator=g, device=dev), torch.tensor([L], dtype=torch.int32, device=dev), None)


CASES = {
    "ties_1m": lambda dev: workloads.gaussian_bf16_ties(1, 1 << 20, seed=1, device=dev) + (2048,),
    "unique_16k": lambda dev: workloads.gaussian_unique(1, 16384, seed=1, device=dev) + (2048,),
    "ties_128k": lambda dev: workloads.gaussian_bf16_ties(1, 131072, seed=1, device=dev) + (2048,),
    "outliers_1m_k512": lambda dev: workloads.gaussian_outliers(1, 1 << 20, seed=1, device=dev) + (512,),
    "long_4m": lambda dev: _gaussian_row(1 << 22, dev) + (2048,),
    "long_8m": lambda dev: _gaussian_row(1 << 23, dev) + (2048,),
    "long_16m": lambda dev: _gaussian_row(1 << 24, dev) + (2048,),
    "ragged_b64": lambda dev: workloads.lightning_indexer_logits(64, 131072, 4096, seed=2, device=dev) + (2048,),
}


def trace_once(score, lengths, k, cluster=0, hinted=False, cold=False):
    """Returns (cluster_size, int64 array [n_ctas, TRACE_SLOTS] of cycle stamps).  With ``hinted`` the
    warm-up launches leave a threshold guess per row and the traced launch uses it (no histogram
    stages then)."""
    lib = _lib.load()
    dev = score.device
    lib.ff_topk_set_cluster_override(cluster)
    import ctypes
    shape = (ctypes.c_int32 * 2)()
    lib.ff_topk_policy_launch_shape(score.shape[0], score.shape[1], k, 1, 1 if hinted else 0, shape)
    C = int(shape[0])            # CTAs per cluster of the launch actually made (a row may span shape[1] clusters)
    # a row may be split over up to 64 clusters of up to 16 CTAs: size the buffer for the largest grid
    buf = torch.zeros((score.shape[0] * 1024, _lib.TRACE_SLOTS), dtype=torch.int64, device=dev)
    out = torch.empty((score.shape[0], k), dtype=torch.int32, device=dev)
    hint = None
    if hinted:
        from . import new_threshold_hint
        hint = new_threshold_hint(score.shape[0], dev)
    for _ in range(3):
        fast_topk_v3(score, lengths, k, out=out, threshold_hint=hint)
    if cold:   # push the row out of L2: the traced launch reads it from HBM, as a decode step would
        torch.empty(256 << 20, dtype=torch.uint8, device=dev).fill_(1)
    torch.cuda.synchronize()
    lib.ff_topk_set_trace_buffer(buf.data_ptr())
    try:
        fast_topk_v3(score, lengths, k, out=out, threshold_hint=hint)
        torch.cuda.synchronize()
    finally:
        lib.ff_topk_set_trace_buffer(None)
        lib.ff_topk_set_cluster_override(0)
    t = buf.cpu().numpy()
    used = int((t[:, 0] != 0).sum())          # CTAs that wrote a start stamp
    return C, t[:max(used, 1)]


def format_timeline(stamps, mhz):
    prev = stamps[0]
    parts = []
    for slot, name in STAGES[1:]:
        if stamps[slot] == 0:
            continue
        parts.append(f"{name} {(stamps[slot] - prev) / mhz:.2f}")
        prev = stamps[slot]
    total = (max(stamps[25], stamps[35]) - stamps[0]) / mhz
    return f"total {total:.2f} us | " + " | ".join(parts)


def trace_context_parallel(mhz: float, shard_columns: int = 1 << 20, k: int = 2048, hinted: bool = False):
    """Under torch.distributed.run (one rank per GPU): a few context-parallel steps on bf16-rounded
    N(0,1) shards, the last one traced.  Every rank reports, over its own CTAs (cycle counters of
    different GPUs are not comparable), when the select was done, how long the merging CTAs then
    waited for the peers' run heads, and how long checking, ranking and writing took."""
    import os
    import torch.distributed as dist
    from . import new_threshold_hint
    from .context_parallel import ContextParallelTopk
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    lib = _lib.load()
    g = torch.Generator(device=dev)
    g.manual_seed(77 + rank)
    shards = torch.randn((8, shard_columns), generator=g, device=dev).to(torch.bfloat16).float()
    lengths = torch.tensor([shard_columns * world], dtype=torch.int32, device=dev)
    buf = torch.zeros((1024, _lib.TRACE_SLOTS), dtype=torch.int64, device=dev)
    hint = new_threshold_hint(1, dev) if hinted else None
    with ContextParallelTopk(1, k, dev) as plan:
        for i in range(6):
            plan(shards[i:i + 1], lengths, rank * shard_columns, threshold_hint=hint)
        torch.cuda.synchronize()
        dist.barrier()
        # ten steps replayed from one CUDA graph, all traced into the same slots: what is read back is
        # the LAST step, taken with the ranks in step with each other (an eager launch would
        # mostly show how far apart the ranks' host threads are)
        lib.ff_topk_set_trace_buffer(buf.data_ptr())
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(10):
                    plan(shards[i % 8:i % 8 + 1], lengths, rank * shard_columns, threshold_hint=hint)
            torch.cuda.synchronize()
            dist.barrier()
            graph.replay()
        torch.cuda.synchronize()
        lib.ff_topk_set_trace_buffer(None)
        plan.check_status()
        t = buf.cpu().numpy()
        t = t[t[:, 0] != 0]
        merging = t[t[:, 35] != 0]
        # the cycle counter is per SM: only differences inside one CTA mean anything
        dur = lambda a, b, rows: (rows[:, b] - rows[:, a]) / mhz
        sel = dur(0, 32, t)
        line = f"rank {rank}: ctas {t.shape[0]} merging {merging.shape[0]} | select (start to select_done) {sel.min():.2f}..{sel.max():.2f}"
        if merging.shape[0]:
            parts = [("wait+stage heads", 36, 33), ("rank own", 33, 37), ("verdict barrier", 37, 34), ("write", 34, 35),
                     ("whole CTA", 0, 35)]
            line += " | merging CTAs (min..max): " + ", ".join(
                f"{n} {dur(a, b, merging).min():.2f}..{dur(a, b, merging).max():.2f}" for n, a, b in parts)
        lines = [None] * world
        dist.all_gather_object(lines, line)
        if rank == 0:
            print(f"== context-parallel step, {world} ranks x {shard_columns} columns, k={k}"
                  f"{' (threshold guesses)' if hinted else ''}, exchange {plan.exchange} (us at {mhz} MHz)")
            for l in lines:
                print("  " + l)
            print(f"  rank 0, first CTA: {format_timeline(t[0], mhz)}")
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cp", action="store_true",
                    help="trace one context-parallel step (run under torch.distributed.run, one rank per GPU)")
    ap.add_argument("--case", default="all", choices=["all"] + sorted(CASES))
    ap.add_argument("--cluster", type=int, default=0)
    ap.add_argument("--mhz", type=float, default=1965.0, help="SM clock used to convert cycles to us")
    ap.add_argument("--hinted", action="store_true", help="trace a launch that uses a threshold guess")
    ap.add_argument("--cold", action="store_true", help="flush L2 before the traced launch")
    args = ap.parse_args()
    if args.cp:
        trace_context_parallel(args.mhz, hinted=args.hinted)
        return
    dev = torch.device("cuda:0")
    mhz = args.mhz
    names = sorted(CASES) if args.case == "all" else [args.case]
    for name in names:
        score, lengths, _, k = CASES[name](dev)
        C, t = trace_once(score, lengths, k, args.cluster, args.hinted, args.cold)
        print(f"== {name}{' (threshold guess)' if args.hinted else ''}{' (cold L2)' if args.cold else ''}: B={score.shape[0]} L={score.shape[1]} k={k} "
              f"cluster={C} ctas={t.shape[0]} (us at {mhz} MHz)")
        for cta in sorted({0, t.shape[0] - 1}):
            print(f"  cta {cta}: {format_timeline(t[cta], mhz)}")
        if (t[:, 7] != 0).all():
            # the own-guess stage on the global timer (ns; comparable between SMs): when, after the
            # first CTA's start, each CTA started, had its sample, sent its estimate, saw all of them
            import numpy as np
            t0 = t[:, 8].min()
            spread = lambda col: "/".join(f"{v / 1e3:.2f}" for v in np.percentile(t[:, col] - t0, [0, 50, 100]))
            print(f"  own guess over all CTAs, us after the first start (min/median/max): start {spread(8)}, "
                  f"sample landed {spread(5)}, estimate sent {spread(6)}, all estimates seen {spread(7)}")


if __name__ == "__main__":
    main()
