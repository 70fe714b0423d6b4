"""Generates tests/golden/topk_golden.npz.

Every expected result is produced by ``torch.sort(descending=True,
stable=True)`` on the window (the definition the reference path is specified
by), and cross-checked here against ``torch.topk`` values.  The reference
repository holds no golden vectors for this path, so these are the pinned
known answers for the oracle and for the CUDA kernels.

Run from the repository root:  python tests/golden/make_golden.py
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from flash_float_jit_kernels_b200 import workloads as W  # noqa: E402


def expected(score, lengths, k, rs):
    B, L = score.shape
    out = torch.full((B, k), -1, dtype=torch.int32)
    for b in range(B):
        s = int(rs[b]) if rs is not None else 0
        n = max(0, min(int(lengths[b]), L - s))
        if n <= k:
            out[b, :n] = torch.arange(n, dtype=torch.int32)
            continue
        win = score[b, s:s + n]
        order = torch.sort(win, descending=True, stable=True).indices[:k]
        tv = torch.topk(win, k, sorted=True).values
        got = win[order]
        same = (tv == got) | (torch.isnan(tv) & torch.isnan(got))
        assert bool(same.all()), "torch.topk values disagree with the stable sort"
        out[b] = order.to(torch.int32)
    return out


def main():
    cases = {}

    def add(name, score, lengths, k, rs=None):
        exp = expected(score, lengths, k, rs)
        cases[f"{name}/score"] = score.numpy()
        cases[f"{name}/lengths"] = lengths.numpy()
        cases[f"{name}/k"] = np.int32(k)
        if rs is not None:
            cases[f"{name}/row_starts"] = rs.numpy()
        cases[f"{name}/expected"] = exp.numpy()

    s, l, _ = W.gaussian_unique(1, 16384, seed=100)
    add("unique_16k_k2048", s, l, 2048)
    s, l, _ = W.gaussian_bf16_ties(2, 8192, seed=101)
    add("bf16_ties_8k_k512", s, l, 512)
    s, l, _ = W.gaussian_outliers(1, 12000, seed=102, frac=0.01)
    add("outliers_12000_k1024", s, l, 1024)
    s, l, _ = W.lightning_indexer_logits(4, 4096, 300, seed=103, heads=8, head_dim=16)
    l[1] = 200   # shorter than k
    l[2] = 512   # exactly k
    s[1, 200:] = float("-inf")
    s[2, 512:] = float("-inf")
    add("ragged_logits_4x4096_k512", s, l, 512)
    for i, dist in enumerate(W.REFERENCE_DISTRIBUTIONS):
        s, l, rs = W.reference_style(2, 3000, True, dist, seed=200 + i, max_seq_len=6000)
        add(f"ref_{dist}_rs_k512", s, l, 512, rs)
    # special values: NaN, infinities, signed zeros, denormals, constant row
    g = torch.Generator().manual_seed(104)
    x = torch.randn((3, 2048), generator=g)
    x[0, ::7] = 0.0
    x[0, 3::7] = -0.0
    x[0, 5] = float("nan")
    x[0, 900] = float("nan")
    x[0, 11] = float("inf")
    x[0, 12] = float("-inf")
    x[0, 13::97] = 1e-42
    x[0, 14::97] = -1e-42
    x[1, :] = 2.5
    x[2, :] = torch.randint(0, 4, (2048,), generator=g).float()
    add("special_values_k64", x, torch.tensor([2048, 2048, 2000], dtype=torch.int32), 64)
    add("special_values_k1000", x, torch.tensor([2048, 2048, 2000], dtype=torch.int32), 1000)
    # 16-bit scores: the expected result is the stable sort of the 16-bit tensor ITSELF; the stored
    # "score" is its exact fp32 widening (what the oracle statements read), "score_bits16" the raw bits
    for tag, dt in (("bf16", torch.bfloat16), ("f16", torch.float16)):
        g = torch.Generator().manual_seed(105)
        x16 = torch.randn((3, 6000), generator=g).to(dt)
        x16[1, 100:200] = 0.0
        x16[1, 150:180] = -0.0
        x16[2, 7] = float("inf")
        x16[2, 8] = float("nan")
        lengths = torch.tensor([6000, 5999, 3001], dtype=torch.int32)
        rs = torch.tensor([0, 1, 2999], dtype=torch.int32)          # odd window starts: misaligned 16-byte units
        for name, k, r in ((f"{tag}_6000_k512", 512, None), (f"{tag}_6000_rs_k1000", 1000, rs)):
            exp = expected(x16, lengths if r is None else torch.tensor([6000, 5999, 3001], dtype=torch.int32), k, r)
            add(name, x16.float(), lengths, k, r)
            assert np.array_equal(cases[f"{name}/expected"], exp.numpy()), "widening changed the order"
            cases[f"{name}/score_bits16"] = x16.view(torch.int16).numpy()
            cases[f"{name}/dtype"] = np.array(tag)
    out = Path(__file__).resolve().parent / "topk_golden.npz"
    np.savez_compressed(out, **cases)
    print(out, out.stat().st_size, "bytes", len([c for c in cases if c.endswith('/k')]), "cases")


if __name__ == "__main__":
    main()
