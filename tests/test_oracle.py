"""The CPU oracle against the pinned golden vectors, and its three statements against each other."""
import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st


def test_golden_has_cases(golden):
    assert len(golden) >= 13


def test_stable_sort_statement_matches_golden(golden, oracle):
    for name, c in golden.items():
        rs = None if c["row_starts"] is None else torch.from_numpy(c["row_starts"])
        got = oracle.topk_stable_sort(torch.from_numpy(c["score"]), torch.from_numpy(c["lengths"]), c["k"], rs)
        assert np.array_equal(got.numpy(), c["expected"]), name


def test_numpy_statement_matches_golden(golden, oracle):
    for name, c in golden.items():
        got = oracle.topk_numpy(c["score"], c["lengths"], c["k"], c["row_starts"])
        assert np.array_equal(got, c["expected"]), name


def test_c_statement_matches_golden(golden, oracle):
    for name, c in golden.items():
        got = oracle.topk_c(c["score"], c["lengths"], c["k"], c["row_starts"])
        assert np.array_equal(got, c["expected"]), name


def test_short_rows_follow_reference_identity_rule(oracle):
    # topk_indexer_radix.cu:180-191: length <= k -> 0..length-1 then -1
    s = np.random.default_rng(0).standard_normal((3, 64)).astype(np.float32)
    lengths = np.array([0, 5, 8], dtype=np.int32)
    got = oracle.topk_c(s, lengths, 8)
    assert got[0].tolist() == [-1] * 8
    assert got[1].tolist() == [0, 1, 2, 3, 4, -1, -1, -1]
    assert got[2].tolist() == list(range(8))


def test_key_map_total_order(oracle):
    vals = np.array([float("-inf"), -3.5, -1e-42, -0.0, 0.0, 1e-42, 1.0, 3.5, float("inf"), float("nan")],
                    dtype=np.float32)
    keys = oracle.monotone_key(vals)
    assert keys[3] == keys[4]                      # -0.0 == +0.0
    assert keys[-1] == 0xFFFFFFFF                  # NaN on top
    nz = [0, 1, 2, 3, 5, 6, 7, 8, 9]
    assert all(keys[a] < keys[b] for a, b in zip(nz, nz[1:]))
    for v, k in zip(vals.view(np.uint32), keys):
        assert oracle.key_c(int(v)) == int(k)
    neg_nan = np.array([0xFFC00001], dtype=np.uint32)
    assert oracle.monotone_key(neg_nan.view(np.float32))[0] == 0xFFFFFFFF


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 400), st.integers(1, 64), st.integers(0, 2**31 - 1), st.sampled_from([2, 5, 1000]))
def test_three_statements_agree(n, k, seed, distinct):
    from oracle import oracle
    rng = np.random.default_rng(seed)
    s = rng.integers(0, distinct, size=(2, n)).astype(np.float32) - distinct / 2
    lengths = np.array([n, max(0, n - 3)], dtype=np.int32)
    a = oracle.topk_c(s, lengths, k)
    b = oracle.topk_numpy(s, lengths, k)
    c = oracle.topk_stable_sort(torch.from_numpy(s), torch.from_numpy(lengths), k).numpy()
    assert np.array_equal(a, b) and np.array_equal(a, c)


def test_transform_statements(oracle):
    rng = np.random.default_rng(3)
    s = rng.standard_normal((4, 300)).astype(np.float32)
    lengths = np.array([300, 10, 250, 300], dtype=np.int32)
    k = 16
    idx = oracle.topk_c(s, lengths, k)
    table = rng.integers(0, 10_000, size=(2, 300)).astype(np.int32)
    cu = np.array([0, 3, 4], dtype=np.int32)
    via_c = oracle.topk_c(s, lengths, k, epilogue=1, table=table, cu_seqlens_q=cu)
    assert np.array_equal(via_c, oracle.transform_page_table(idx, table, cu))
    off = np.array([7, 100, -5, 0], dtype=np.int32)
    via_c = oracle.topk_c(s, lengths, k, epilogue=2, offsets=off)
    assert np.array_equal(via_c, oracle.transform_ragged(idx, off))


@pytest.mark.parametrize("P", [1, 2, 3, 8])
def test_cp_statement_equals_unsharded(oracle, P):
    from flash_float_jit_kernels_b200.context_parallel import shard_bounds
    rng = np.random.default_rng(P)
    B, L, k = 3, 5000, 128
    s = rng.integers(-50, 50, size=(B, L)).astype(np.float32)  # heavy ties
    lengths = np.array([L, 100, 4097], dtype=np.int32)
    vals, idxs = [], []
    for r in range(P):
        a, b = shard_bounds(L, P, r)
        v, g = oracle.cp_local(np.ascontiguousarray(s[:, a:b]), lengths, k, a)
        vals.append(v)
        idxs.append(g)
    got = oracle.cp_merge(np.stack(vals), np.stack(idxs), lengths, k)
    assert np.array_equal(got, oracle.topk_c(s, lengths, k))
