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
    (0, "start"), (1, "sweep1_hist"), (26, "merge_barrier"), (27, "merge_remote_loads"),
    (28, "merge_scan"), (29, "merge_fine_loads"), (30, "merge_threshold"), (2, "merge_end"),
    (3, "sweep2_collect"), (4, "gather_to_peers"), (20, "final_barrier"), (22, "finish_bin_hist"),
    (23, "finish_scan"), (24, "finish_scatter"), (31, "finish_queue_units"), (25, "finish_rank_emit"),
]

CASES = {
    "ties_1m": lambda dev: workloads.gaussian_bf16_ties(1, 1 << 20, seed=1, device=dev) + (2048,),
    "unique_16k": lambda dev: workloads.gaussian_unique(1, 16384, seed=1, device=dev) + (2048,),
    "ties_128k": lambda dev: workloads.gaussian_bf16_ties(1, 131072, seed=1, device=dev) + (2048,),
    "outliers_1m_k512": lambda dev: workloads.gaussian_outliers(1, 1 << 20, seed=1, device=dev) + (512,),
    "ragged_b64": lambda dev: workloads.lightning_indexer_logits(64, 131072, 4096, seed=2, device=dev) + (2048,),
}


def trace_once(score, lengths, k, cluster=0, hinted=False):
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
    total = (stamps[25] - stamps[0]) / mhz
    return f"total {total:.2f} us | " + " | ".join(parts)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all", choices=["all"] + sorted(CASES))
    ap.add_argument("--cluster", type=int, default=0)
    ap.add_argument("--mhz", type=float, default=1965.0, help="SM clock used to convert cycles to us")
    ap.add_argument("--hinted", action="store_true", help="trace a launch that uses a threshold guess")
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    mhz = args.mhz
    names = sorted(CASES) if args.case == "all" else [args.case]
    for name in names:
        score, lengths, _, k = CASES[name](dev)
        C, t = trace_once(score, lengths, k, args.cluster, args.hinted)
        print(f"== {name}{' (threshold guess)' if args.hinted else ''}: B={score.shape[0]} L={score.shape[1]} k={k} "
              f"cluster={C} ctas={t.shape[0]} (us at {mhz} MHz)")
        for cta in sorted({0, t.shape[0] - 1}):
            print(f"  cta {cta}: {format_timeline(t[cta], mhz)}")


if __name__ == "__main__":
    main()
