"""Lightning-indexer logit producer (tcgen05 kernel): ABI checks on CPU, bit-exact parity on a GPU."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def _declared():
    text = (ROOT / "include" / "ff_indexer_logits.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ff_[a-z0-9_]+)\s*\(", text)))


def test_library_loads_and_exports_every_declared_symbol():
    from flash_float_jit_kernels_b200 import build, indexer_logits
    build.build_indexer_library()
    lib = indexer_logits.load()
    raw = ctypes.CDLL(str(build.indexer_lib_path()))
    names = _declared()
    assert "ff_indexer_logits_launch" in names
    for name in names:
        assert hasattr(raw, name), f"{name} declared but not exported"
        assert name in indexer_logits.SIGNATURES
    # argument validation needs no GPU
    assert lib.ff_indexer_logits_launch(None, None, 0, None, None, None, 0, -1, 8, 0, None, None) == -2
    assert lib.ff_indexer_logits_launch(None, None, 0, None, None, None, 0, 1, 8, 0, None, None) == -3
    assert lib.ff_indexer_logits_launch(None, None, 0, None, None, None, 0, 0, 8, 0, None, None) == 0


def test_oracle_logits_agree_with_a_plain_matmul(oracle):
    g = torch.Generator().manual_seed(0)
    q = (torch.randn((64, 128), generator=g) / 4).to(torch.float8_e4m3fn).float()
    k = (torch.randn((500, 128), generator=g) / 4).to(torch.float8_e4m3fn).float()
    w = torch.rand((64,), generator=g)
    s, inexact = oracle.indexer_logits(q.numpy(), k.numpy(), w.numpy())
    assert inexact == 0          # every dot product is exact in float32 for this distribution
    ref = (torch.relu(k @ q.t()) @ w).numpy()
    assert np.allclose(s, ref, rtol=1e-5, atol=1e-5)


def _make(B, L, seed, device):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn((B, 64, 128), generator=g) / 4).to(torch.float8_e4m3fn)
    k = (torch.randn((B, L, 128), generator=g) / 4).to(torch.float8_e4m3fn)
    w = torch.rand((B, 64), generator=g)
    return q, k, w


@pytest.mark.gpu
@pytest.mark.parametrize("B,L,lens,ctas", [(1, 128, [128], 1), (2, 1000, [1000, 37], 0), (3, 5000, [5000, 4097, 129], 3),
                                           (2, 20000, [20000, 1], -1), (5, 3000, [3000, 0, 129, 2999, 1024], -1), (5, 3000, [3000, 0, 129, 2999, 1024], 0),
                                           (70, 2100, [2100 - 29 * i for i in range(70)], -1)])
def test_logits_are_bit_exact_against_the_oracle(oracle, B, L, lens, ctas):
    from flash_float_jit_kernels_b200.indexer_logits import indexer_logits_fp8
    dev = torch.device("cuda:0")
    q, k, w = _make(B, L, 11 + L, dev)
    lengths = torch.tensor(lens, dtype=torch.int32)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = indexer_logits_fp8(q.to(dev), k.to(dev), w.to(dev), lengths.to(dev), status=status, ctas_per_row=ctas)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got = out.cpu().numpy()
    for b in range(B):
        n = lens[b]
        exp, inexact = oracle.indexer_logits(q[b].float().numpy(), k[b, :n].float().numpy(), w[b].numpy())
        assert inexact == 0
        assert np.array_equal(got[b, :n].view(np.uint32), exp.view(np.uint32)), (
            b, float(np.abs(got[b, :n] - exp).max()))
        assert np.all(np.isneginf(got[b, n:]))


@pytest.mark.gpu
def test_logits_feed_the_indexer(oracle):
    """Producer and selector back to back: the top-k of the produced scores is the oracle's
    top-k of the oracle's scores."""
    from flash_float_jit_kernels_b200 import fast_topk_v3
    from flash_float_jit_kernels_b200.indexer_logits import indexer_logits_fp8
    dev = torch.device("cuda:0")
    B, L, k_top = 2, 9000, 512
    q, k, w = _make(B, L, 5, dev)
    lengths = torch.tensor([9000, 6001], dtype=torch.int32)
    scores = indexer_logits_fp8(q.to(dev), k.to(dev), w.to(dev), lengths.to(dev))
    idx = fast_topk_v3(scores, lengths.to(dev), k_top)
    torch.cuda.synchronize()
    exp_scores = np.full((B, L), -np.inf, dtype=np.float32)
    for b in range(B):
        n = int(lengths[b])
        exp_scores[b, :n] = oracle.indexer_logits(q[b].float().numpy(), k[b, :n].float().numpy(), w[b].numpy())[0]
    assert np.array_equal(idx.cpu().numpy(), oracle.topk_c(exp_scores, lengths.numpy(), k_top))


@pytest.mark.gpu
def test_decode_step_with_threshold_guesses(oracle):
    """indexer_topk over a few steps of a growing K cache, guesses carried along: exact every step."""
    from flash_float_jit_kernels_b200 import new_threshold_hint
    from flash_float_jit_kernels_b200.indexer_logits import indexer_topk
    dev = torch.device("cuda:0")
    B, L, k_top = 2, 12000, 256
    q, k, w = _make(B, L, 21, dev)
    qd, kd, wd = q.to(dev), k.to(dev), w.to(dev)
    scores = torch.full((B, L), float("-inf"), device=dev)
    out = torch.empty((B, k_top), dtype=torch.int32, device=dev)
    hint = new_threshold_hint(B, dev)
    for step in range(3):
        lengths = torch.tensor([11000 + 300 * step, 7000 + 100 * step], dtype=torch.int32)
        indexer_topk(qd, kd, wd, lengths.to(dev), k_top, scores=scores, out=out, threshold_hint=hint)
        torch.cuda.synchronize()
        exp_scores = np.full((B, L), -np.inf, dtype=np.float32)
        for b in range(B):
            n = int(lengths[b])
            exp_scores[b, :n] = oracle.indexer_logits(q[b].float().numpy(), k[b, :n].float().numpy(), w[b].numpy())[0]
        assert np.array_equal(out.cpu().numpy(), oracle.topk_c(exp_scores, lengths.numpy(), k_top)), step


@pytest.mark.gpu
@pytest.mark.parametrize("B,L,k_top", [(3, 40000, 512), (1, 300000, 2048), (64, 16384, 1024)])
def test_decode_steps_with_survivor_hand_over(oracle, B, L, k_top):
    """The producer lists every score not below the row's guess; a row whose guess fits is ranked
    from the list alone.  Steps: no guess yet (lists empty, select from the scores), guesses hit
    (same queries), a jump (too many listed: miss, select from the scores), hit again; one row
    is at times no longer than k.  Exact every step; the list headers come back zeroed."""
    from flash_float_jit_kernels_b200 import _lib, new_threshold_hint
    from flash_float_jit_kernels_b200.indexer_logits import indexer_topk, new_handover
    dev = torch.device("cuda:0")
    q, k, w = _make(B, L, 31 + B, dev)
    kd, wd = k.to(dev), w.to(dev)
    scores = torch.full((B, L), float("-inf"), device=dev)
    out = torch.empty((B, k_top), dtype=torch.int32, device=dev)
    hint = new_threshold_hint(B, dev)
    handover = new_handover(B, dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    kf = k.float().numpy()
    seen = []
    for step in range(5):
        qs = q.float()
        if step >= 3:
            qs = qs * 2.0                      # every score doubles (and stays so): the old guesses let far too many through
        qs = qs.to(torch.float8_e4m3fn)
        lens = [L - 128 * step - 5] + [max(k_top + 1, L // (2 + b)) + 64 * step for b in range(1, B)]
        if B > 1 and step in (2, 4):
            lens[1] = k_top - 3                # a row no longer than k: identity order, its list header is cleared
        lengths = torch.tensor(lens, dtype=torch.int32)
        status.zero_()
        indexer_topk(qs.to(dev), kd, wd, lengths.to(dev), k_top, scores=scores, out=out, threshold_hint=hint,
                     status=status, handover=handover)
        torch.cuda.synchronize()
        seen.append(int(status.item()))
        exp_scores = np.full((B, L), -np.inf, dtype=np.float32)
        for b in range(min(B, 4)):             # the oracle's own scores for the first rows, the produced ones for the rest
            n = lens[b]
            exp_scores[b, :n] = oracle.indexer_logits(qs[b].float().numpy(), kf[b, :n], w[b].numpy())[0]
        got_scores = scores.cpu().numpy()
        for b in range(4, B):
            exp_scores[b, :lens[b]] = got_scores[b, :lens[b]]
        assert np.array_equal(out.cpu().numpy(), oracle.topk_c(exp_scores, lengths.numpy(), k_top)), step
        hdr = handover.view(torch.int32).view(B, _lib.FF_TOPK_HANDOVER_ROW_BYTES // 4)[:, :2].cpu()
        assert int(hdr.abs().sum()) == 0, f"step {step}: list headers not cleared: {hdr.tolist()[:4]}"
    assert seen[0] == 0, "no guesses yet: nothing can miss"
    assert seen[1] == 0, "guesses from the first step fit the second"
    assert seen[3] == _lib.FF_STATUS_HINT_MISSED, "doubled scores: the lists overflow, the select falls back"
    assert seen[4] == 0
