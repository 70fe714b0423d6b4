"""Seeded synthetic score generators for tests and benchmarks.

They stand in for real indexer logits: the five benchmark configurations
(unique Gaussian, bf16-rounded Gaussian with heavy ties, ragged
lightning-indexer logits, Gaussian with an outlier tail, long rows for the
context-parallel mode) and the reference benchmark's seven ``[0, 255]``-scaled
distributions (``benchmark/bench_topk.py:60-125``).  Everything is drawn from
a ``torch.Generator`` with a fixed seed on the requested device, so CPU and
GPU runs of a test see the tensor they generated themselves (the oracle always
receives a copy of the very tensor the kernel reads).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

Triple = Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _full_lengths(B: int, L: int, device) -> torch.Tensor:
    return torch.full((B,), L, dtype=torch.int32, device=device)


def gaussian_unique(B: int, L: int, seed: int = 0, device="cpu") -> Triple:
    """i.i.d. N(0,1) with duplicates resampled until every value in a row is unique."""
    g = _gen(seed, device)
    x = torch.randn((B, L), generator=g, device=device, dtype=torch.float32)
    for b in range(B):
        for _ in range(64):
            s, order = torch.sort(x[b])
            dup = torch.zeros(L, dtype=torch.bool, device=device)
            dup[1:] = s[1:] == s[:-1]
            n = int(dup.sum())
            if n == 0:
                break
            x[b, order[dup]] = torch.randn((n,), generator=g, device=device, dtype=torch.float32)
    return x, _full_lengths(B, L, device), None


def gaussian_bf16_ties(B: int, L: int, seed: int = 1, device="cpu") -> Triple:
    """N(0,1) rounded to bf16 and cast back: ~90 duplicates per value near the top-2048 threshold at L=1M."""
    g = _gen(seed, device)
    x = torch.randn((B, L), generator=g, device=device, dtype=torch.float32)
    return x.to(torch.bfloat16).to(torch.float32), _full_lengths(B, L, device), None


def gaussian_outliers(B: int, L: int, seed: int = 3, device="cpu", frac: float = 1e-3) -> Triple:
    """99.9 % N(0,1) + 0.1 % N(6,1) at seeded positions (one dominant tail)."""
    g = _gen(seed, device)
    x = torch.randn((B, L), generator=g, device=device, dtype=torch.float32)
    mask = torch.rand((B, L), generator=g, device=device) < frac
    out = torch.randn((B, L), generator=g, device=device, dtype=torch.float32) + 6.0
    return torch.where(mask, out, x), _full_lengths(B, L, device), None


def lightning_indexer_logits(B: int, L_max: int, min_len: int, seed: int = 2, device="cpu",
                             heads: int = 64, head_dim: int = 128, chunk: int = 16384) -> Triple:
    """Ragged decode batch: ``s[j] = sum_h w_h * relu(q_h . k_j)`` with q, K drawn
    N(0,1)/4 and rounded to fp8 e4m3, w ~ U(0,1), fp32 accumulation; positions
    beyond the row's length hold ``-inf``; lengths ~ U{min_len..L_max}."""
    g = _gen(seed, device)
    lengths = torch.randint(min_len, L_max + 1, (B,), generator=g, device=device, dtype=torch.int32)
    scores = torch.full((B, L_max), float("-inf"), device=device, dtype=torch.float32)
    f8 = torch.float8_e4m3fn
    for b in range(B):
        n = int(lengths[b])
        q = (torch.randn((heads, head_dim), generator=g, device=device) / 4).to(f8).to(torch.float32)
        w = torch.rand((heads,), generator=g, device=device, dtype=torch.float32)
        for s in range(0, n, chunk):
            e = min(n, s + chunk)
            kk = (torch.randn((e - s, head_dim), generator=g, device=device) / 4).to(f8).to(torch.float32)
            logits = torch.relu(kk @ q.t())          # [chunk, heads], fp32 accumulate
            scores[b, s:e] = logits @ w
    return scores, lengths, None


# ---- the reference benchmark's distributions, scaled to [0, 255] -----------
def _ref_unit(dist: str, n: int, g: torch.Generator, device) -> torch.Tensor:
    """The seven [0, 1] score distributions of the reference benchmark, with its parameters
    (``benchmark/bench_topk.py:60-96``), drawn from a seeded generator instead of the global one."""
    def randn():
        return torch.randn((n,), generator=g, device=device, dtype=torch.float32)

    def rand():
        return torch.rand((n,), generator=g, device=device, dtype=torch.float32)

    if dist == "gaussian":      # randn normalised by its own range (+1e-6), bench_topk.py:86-89
        x = randn()
        return (x - x.min()) / (x.max() - x.min() + 1e-6)
    if dist == "uniform":       # bench_topk.py:60-61
        return rand()
    if dist == "sigmoid":       # sigmoid of a standard normal, bench_topk.py:64-66
        return torch.sigmoid(randn())
    if dist == "beta":          # Beta(0.5, 0.5), bench_topk.py:69-71; drawn by the arcsine law sin^2(pi/2 U),
        return torch.sin(rand() * (math.pi / 2)) ** 2      # which has exactly that distribution
    if dist == "power":         # U^6, bench_topk.py:74-76
        return rand() ** 6
    if dist == "bimodal":       # half uniform on [0, 0.25], half uniform on [0.75, 1], bench_topk.py:79-83
        pick = rand() < 0.5
        return torch.where(pick, 0.25 * rand(), 0.75 + 0.25 * rand())
    if dist == "sparse":        # 2 % spikes uniform on [0.5, 1], background uniform on [0, 0.01], bench_topk.py:92-96
        hot = rand() < 0.02
        return torch.where(hot, 0.5 + 0.5 * rand(), 0.01 * rand())
    raise ValueError(dist)


REFERENCE_DISTRIBUTIONS = ("gaussian", "uniform", "sigmoid", "beta", "power", "bimodal", "sparse")
# the reference benchmark's grid (bench_topk.py:418-431): every combination, each with and without row_starts
REFERENCE_GRID_BS = (1, 2, 4, 8)
REFERENCE_GRID_K = (512, 1024, 2048)
REFERENCE_GRID_SEQ_LEN = (16384, 65536, 98304, 120000)


def reference_style(B: int, seq_len: int, has_row_starts: bool, dist: str = "uniform",
                    seed: int = 42, device="cpu", max_seq_len: int = 131072) -> Triple:
    """Scores in [0, 255] the way the reference benchmark builds them
    (``bench_topk.py:111-125``): tensor width ``max_seq_len`` and random
    ``row_starts`` in [0, 2048) when ``has_row_starts``."""
    g = _gen(seed, device)
    L = max_seq_len if has_row_starts else seq_len
    x = _ref_unit(dist, B * L, g, device).reshape(B, L).clamp(0.0, 1.0) * 255.0
    lengths = torch.full((B,), seq_len, dtype=torch.int32, device=device)
    rs = None
    if has_row_starts:
        rs = torch.randint(0, 2048, (B,), generator=g, device=device, dtype=torch.int32)
    return x, lengths, rs
