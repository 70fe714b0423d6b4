"""Parity of the CUDA top-k (called through the C ABI) with the CPU oracle: bit-exact int32 indices."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

CLUSTERS = [1, 2, 4, 8, 16]


@pytest.fixture(scope="module")
def ff():
    import flash_float_jit_kernels_b200 as pkg
    from flash_float_jit_kernels_b200 import _lib
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    lib = _lib.load()           # raises if the CUDA library is missing: no fallback
    assert lib.ff_topk_init(0) == 0
    yield pkg, lib
    lib.ff_topk_set_cluster_override(0)


def run_case(ff, oracle, score_cpu, lengths_cpu, k, rs_cpu=None, cluster=0, score_dev=None):
    pkg, lib = ff
    assert lib.ff_topk_set_cluster_override(cluster) == 0
    dev = torch.device("cuda:0")
    s = score_cpu.to(dev) if score_dev is None else score_dev
    l = lengths_cpu.to(dev)
    rs = None if rs_cpu is None else rs_cpu.to(dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    before = lib.ff_topk_launch_count()
    out = pkg.fast_topk_v3(s, l, k, rs, status=status)
    torch.cuda.synchronize()
    assert lib.ff_topk_launch_count() == before + 1
    assert int(status.item()) == 0, f"device status {int(status.item())}"
    exp = oracle.topk_c(score_cpu.numpy(), lengths_cpu.numpy(), k, None if rs_cpu is None else rs_cpu.numpy())
    got = out.cpu().numpy()
    if not np.array_equal(got, exp):
        bad = np.argwhere(got != exp)
        raise AssertionError(f"mismatch at {bad[:5].tolist()} of {len(bad)}; got {got[tuple(bad[0])]} want {exp[tuple(bad[0])]}")
    return out


@pytest.mark.parametrize("cluster", CLUSTERS)
def test_golden_vectors(ff, oracle, golden, cluster):
    pkg, lib = ff
    lib.ff_topk_set_cluster_override(cluster)
    for name, c in golden.items():
        s = torch.from_numpy(c["score"]).cuda()
        l = torch.from_numpy(c["lengths"]).cuda()
        rs = None if c["row_starts"] is None else torch.from_numpy(c["row_starts"]).cuda()
        out = pkg.fast_topk_v3(s, l, c["k"], rs)
        assert np.array_equal(out.cpu().numpy(), c["expected"]), f"{name} cluster={cluster}"


@pytest.mark.parametrize("cluster", [0, 1, 4, 16])
def test_config1_unique_gaussian_16k(ff, oracle, cluster):
    from flash_float_jit_kernels_b200 import workloads as W
    s, l, _ = W.gaussian_unique(1, 16384, seed=0)
    run_case(ff, oracle, s, l, 2048, cluster=cluster)


@pytest.mark.parametrize("L", [65536, 131072, 262144, 524288, 1048576])
def test_config2_bf16_ties_latency_sweep(ff, oracle, L):
    from flash_float_jit_kernels_b200 import workloads as W
    s, l, _ = W.gaussian_bf16_ties(1, L, seed=1)
    run_case(ff, oracle, s, l, 2048)


def test_config3_ragged_lightning_logits_b64(ff, oracle):
    from flash_float_jit_kernels_b200 import workloads as W
    s, l, _ = W.lightning_indexer_logits(64, 131072, 4096, seed=2, device="cuda")
    run_case(ff, oracle, s.cpu(), l.cpu(), 2048, score_dev=s)


@pytest.mark.parametrize("B,k", [(1, 512), (1, 1024), (4, 512), (4, 1024)])
def test_config4_outlier_tail_small_k(ff, oracle, B, k):
    from flash_float_jit_kernels_b200 import workloads as W
    s, l, _ = W.gaussian_outliers(B, 1048576, seed=3)
    run_case(ff, oracle, s, l, k)


@pytest.mark.parametrize("L", [4194304, 8388608])
def test_config5_long_rows_single_gpu(ff, oracle, L):
    s = torch.randn((1, L), generator=torch.Generator().manual_seed(5))
    run_case(ff, oracle, s, torch.tensor([L], dtype=torch.int32), 2048)


@pytest.mark.parametrize("dist", ["gaussian", "uniform", "sigmoid", "beta", "power", "bimodal", "sparse"])
@pytest.mark.parametrize("has_rs", [False, True])
def test_reference_benchmark_distributions(ff, oracle, dist, has_rs):
    # every distribution of benchmark/bench_topk.py:60-96 on four points of its grid
    from flash_float_jit_kernels_b200 import workloads as W
    for bs, k, seq in [(1, 2048, 16384), (2, 512, 65536), (4, 1024, 98304), (8, 2048, 120000)]:
        s, l, rs = W.reference_style(bs, seq, has_rs, dist, seed=42)
        run_case(ff, oracle, s, l, k, rs)


@pytest.mark.parametrize("has_rs", [False, True])
@pytest.mark.parametrize("bs", [1, 2, 4, 8])
def test_reference_benchmark_whole_grid(ff, oracle, bs, has_rs):
    # the whole (bs, k, seq_len, has_row_starts) grid of benchmark/bench_topk.py:418-431 on the
    # distribution that benchmark runs ("gaussian", bench_topk.py:437)
    from flash_float_jit_kernels_b200 import workloads as W
    assert bs in W.REFERENCE_GRID_BS
    for seq in W.REFERENCE_GRID_SEQ_LEN:
        s, l, rs = W.reference_style(bs, seq, has_rs, "gaussian", seed=42 + seq)
        sd = s.cuda()
        for k in W.REFERENCE_GRID_K:
            run_case(ff, oracle, s, l, k, rs, score_dev=sd)


@pytest.mark.parametrize("cluster", CLUSTERS)
@pytest.mark.parametrize("L,k", [(2049, 2048), (2079, 2048), (4097, 512), (513, 512), (7919, 1024), (33, 32), (2, 1),
                                 (100003, 2048), (65537, 1)])
def test_edge_lengths(ff, oracle, cluster, L, k):
    g = torch.Generator().manual_seed(L * 31 + k)
    s = torch.randn((3, L), generator=g)
    lengths = torch.tensor([L, max(0, L - 1), L // 2], dtype=torch.int32)
    run_case(ff, oracle, s, lengths, k, cluster=cluster)


@pytest.mark.parametrize("cluster", [1, 2, 16])
def test_short_and_empty_rows(ff, oracle, cluster):
    s = torch.randn((5, 4096), generator=torch.Generator().manual_seed(7))
    lengths = torch.tensor([0, 1, 511, 512, 4096], dtype=torch.int32)
    out = run_case(ff, oracle, s, lengths, 512, cluster=cluster)
    assert out[0].tolist() == [-1] * 512
    assert out[3].tolist() == list(range(512))


@pytest.mark.parametrize("cluster", [1, 4, 16])
def test_all_equal_and_few_distinct_rows(ff, oracle, cluster):
    # every element lands in the threshold bin: candidate buffers overflow and the
    # select must continue into the index bits without dropping anything
    L = 300000
    s = torch.empty((4, L))
    s[0] = 1.25
    s[1] = torch.randint(0, 3, (L,), generator=torch.Generator().manual_seed(1)).float()
    s[2] = float("-inf")
    s[3] = torch.arange(L, dtype=torch.float32)          # sorted ascending: all winners in the last chunk
    lengths = torch.tensor([L, L, L, L], dtype=torch.int32)
    for k in (1, 512, 2048):
        run_case(ff, oracle, s, lengths, k, cluster=cluster)


def test_special_values(ff, oracle):
    g = torch.Generator().manual_seed(11)
    s = torch.randn((2, 50000), generator=g)
    s[0, ::5] = 0.0
    s[0, 1::5] = -0.0
    s[0, 2::1000] = float("nan")
    s[0, 3::1000] = float("inf")
    s[0, 4::1000] = float("-inf")
    s[0].view(torch.int32)[7::1000] = -4194304 + 5       # negative NaN with a payload (0xFFC00005)
    s[0].view(torch.int32)[8::1000] = 0x7F800001          # signalling NaN
    s[1] = s[1].abs() * 1e-42                            # denormals
    lengths = torch.tensor([50000, 50000], dtype=torch.int32)
    for k in (16, 512, 2048):
        run_case(ff, oracle, s, lengths, k)


@pytest.mark.parametrize("cluster", [1, 2, 8])
def test_misaligned_windows_and_row_stride(ff, oracle, cluster):
    g = torch.Generator().manual_seed(13)
    base = torch.randn((6, 70001), generator=g)          # odd row stride: rows start at every alignment
    rs = torch.tensor([0, 1, 2, 3, 5, 4099], dtype=torch.int32)
    lengths = torch.tensor([65000, 64999, 30001, 2050, 513, 60000], dtype=torch.int32)
    run_case(ff, oracle, base, lengths, 512, rs, cluster=cluster)
    view = base[:, 3:60003]                              # non-contiguous view, stride(0) != size(1)
    dev_view = base.cuda()[:, 3:60003]
    pkg, lib = ff
    lib.ff_topk_set_cluster_override(cluster)
    l2 = torch.tensor([60000, 59999, 100, 2050, 513, 60000], dtype=torch.int32)
    out = pkg.fast_topk_v3(dev_view, l2.cuda(), 2048)
    exp = oracle.topk_c(np.ascontiguousarray(view.numpy()), l2.numpy(), 2048)
    assert np.array_equal(out.cpu().numpy(), exp)


def test_lengths_beyond_width_are_clamped(ff, oracle):
    s = torch.randn((2, 5000), generator=torch.Generator().manual_seed(17))
    lengths = torch.tensor([9999, -5], dtype=torch.int32)
    run_case(ff, oracle, s, lengths, 64)


def test_every_k_from_1_to_40_and_odd_k(ff, oracle):
    s = torch.randn((1, 30000), generator=torch.Generator().manual_seed(19))
    l = torch.tensor([30000], dtype=torch.int32)
    for k in list(range(1, 41)) + [100, 777, 1500, 2047]:
        run_case(ff, oracle, s, l, k)


def test_determinism_three_runs(ff):
    pkg, lib = ff
    lib.ff_topk_set_cluster_override(0)
    from flash_float_jit_kernels_b200 import workloads as W
    s, l, _ = W.gaussian_bf16_ties(4, 262144, seed=23, device="cuda")
    outs = [pkg.fast_topk_v3(s, l, 2048).clone() for _ in range(3)]
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_full_size_properties_without_the_oracle(ff):
    # size-independent checks at the largest configuration: selected values are exactly
    # the k largest (checked against a value threshold count) and the order is canonical
    pkg, lib = ff
    lib.ff_topk_set_cluster_override(0)
    L, k = 8388608, 2048
    s = torch.randn((1, L), generator=torch.Generator(device="cuda").manual_seed(29), device="cuda")
    idx = pkg.fast_topk_v3(s, torch.tensor([L], dtype=torch.int32, device="cuda"), k)[0].long()
    v = s[0, idx]
    assert bool((v[:-1] >= v[1:]).all())
    ties = v[:-1] == v[1:]
    assert bool((idx[:-1][ties] < idx[1:][ties]).all())
    assert idx.unique().numel() == k
    thr = v[-1]
    assert int((s[0] > thr).sum()) <= k - 1 < int((s[0] >= thr).sum())


def test_cuda_graph_capture_and_replay(ff, oracle):
    pkg, lib = ff
    lib.ff_topk_set_cluster_override(0)
    from flash_float_jit_kernels_b200 import workloads as W
    s, l, _ = W.gaussian_bf16_ties(2, 100000, seed=31, device="cuda")
    out = torch.empty((2, 1024), dtype=torch.int32, device="cuda")
    pkg.fast_topk_v3(s, l, 1024, out=out)               # warm-up outside capture (one-time set-up)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        pkg.fast_topk_v3(s, l, 1024, out=out)
    s2, _, _ = W.gaussian_bf16_ties(2, 100000, seed=32, device="cuda")
    s.copy_(s2)
    graph.replay()
    torch.cuda.synchronize()
    exp = oracle.topk_c(s.cpu().numpy(), l.cpu().numpy(), 1024)
    assert np.array_equal(out.cpu().numpy(), exp)


def test_transform_page_table_and_ragged(ff, oracle):
    pkg, lib = ff
    lib.ff_topk_set_cluster_override(0)
    g = torch.Generator().manual_seed(37)
    B, L, k = 6, 20000, 2048
    s = torch.randn((B, L), generator=g)
    lengths = torch.tensor([20000, 1000, 19999, 2048, 2049, 20000], dtype=torch.int32)
    idx = oracle.topk_c(s.numpy(), lengths.numpy(), k)
    # decode: one request per row
    table = torch.randint(0, 1 << 20, (B, L), generator=g, dtype=torch.int32)
    cu = torch.arange(B + 1, dtype=torch.int32)
    dst = torch.empty((B, k), dtype=torch.int32, device="cuda")
    pkg.fast_topk_transform_fused(s.cuda(), lengths.cuda(), dst, table.cuda(), cu.cuda())
    assert np.array_equal(dst.cpu().numpy(), oracle.transform_page_table(idx, table.numpy(), None))
    # prefill: 3 requests expanded to 6 rows, with row_starts
    cu = torch.tensor([0, 2, 3, 6], dtype=torch.int32)
    table = torch.randint(0, 1 << 20, (3, L), generator=g, dtype=torch.int32)
    rs = torch.tensor([0, 3, 17, 0, 1, 2], dtype=torch.int32)
    l2 = torch.tensor([19000, 1000, 19983, 2048, 2049, 19998], dtype=torch.int32)
    idx2 = oracle.topk_c(s.numpy(), l2.numpy(), k, rs.numpy())
    pkg.fast_topk_transform_fused(s.cuda(), l2.cuda(), dst, table.cuda(), cu.cuda(), rs.cuda())
    assert np.array_equal(dst.cpu().numpy(), oracle.transform_page_table(idx2, table.numpy(), cu.numpy()))
    # ragged offsets
    off = torch.tensor([0, 20000, 21000, 40999, 43047, 45096], dtype=torch.int32)
    pkg.fast_topk_transform_ragged_fused(s.cuda(), l2.cuda(), dst, off.cuda(), rs.cuda())
    assert np.array_equal(dst.cpu().numpy(), oracle.transform_ragged(idx2, off.numpy()))


# ---- rows split over several clusters (global scratch + row-wide barriers) ----------------
def run_grouped(ff, oracle, s, lengths, k, cluster, groups, rs=None, repeat=2):
    pkg, lib = ff
    assert lib.ff_topk_set_cluster_override(cluster) == 0
    assert lib.ff_topk_set_groups_override(groups) == 0
    try:
        sd, ld = s.cuda(), lengths.cuda()
        rsd = None if rs is None else rs.cuda()
        exp = oracle.topk_c(s.numpy(), lengths.numpy(), k, None if rs is None else rs.numpy())
        for _ in range(repeat):                      # the scratch must come back zeroed
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            out = pkg.fast_topk_v3(sd, ld, k, rsd, status=status)
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            assert np.array_equal(out.cpu().numpy(), exp), f"cluster={cluster} groups={groups}"
    finally:
        lib.ff_topk_set_groups_override(0)
        lib.ff_topk_set_cluster_override(0)


@pytest.mark.parametrize("cluster,groups", [(1, 2), (2, 3), (4, 5), (8, 4), (8, 16), (16, 2), (1, 64)])
def test_rows_split_over_clusters(ff, oracle, cluster, groups):
    g = torch.Generator().manual_seed(41)
    s = torch.randn((2, 300001), generator=g).to(torch.bfloat16).float()
    lengths = torch.tensor([300001, 123457], dtype=torch.int32)
    for k in (512, 2048):
        run_grouped(ff, oracle, s, lengths, k, cluster, groups)


def test_split_rows_automatic_policy_at_full_size(ff, oracle):
    from flash_float_jit_kernels_b200 import workloads as W
    for L in (1 << 20, 1 << 22):
        s, l, _ = W.gaussian_bf16_ties(1, L, seed=43)
        run_grouped(ff, oracle, s, l, 2048, 0, 0)
    s, l, _ = W.gaussian_outliers(4, 1 << 20, seed=44)
    run_grouped(ff, oracle, s, l, 512, 0, 0)


def test_very_long_rows(ff, oracle):
    """32 Mi columns and a ragged length just below: 17 tiles per CTA, counts beyond 2^24 per histogram."""
    g = torch.Generator().manual_seed(99)
    L = 1 << 25
    s = torch.randn((1, L), generator=g)
    for length, k in ((L, 2048), (L - 12345, 512)):
        run_grouped(ff, oracle, s, torch.tensor([length], dtype=torch.int32), k, 0, 0)
    s = s.to(torch.bfloat16).float()                                # heavy ties: about 3000 equal scores per value
    run_grouped(ff, oracle, s, torch.tensor([L], dtype=torch.int32), 2048, 0, 0)


@pytest.mark.parametrize("cluster,groups", [(8, 4), (2, 7)])
def test_split_rows_deeper_levels_and_ties(ff, oracle, cluster, groups):
    L = 400000
    s = torch.empty((4, L))
    s[0] = 1.25                                                    # every element in one bin, all levels
    s[1] = torch.rand((L,), generator=torch.Generator().manual_seed(2)) * 255.0   # coarse bins: second level
    s[2] = torch.arange(L, dtype=torch.float32)                    # all winners in the last chunk
    s[3] = torch.randint(0, 3, (L,), generator=torch.Generator().manual_seed(3)).float()
    lengths = torch.tensor([L, L, L, L - 5], dtype=torch.int32)
    rs = torch.tensor([0, 1, 2, 3], dtype=torch.int32)
    run_grouped(ff, oracle, s, lengths - 3, 2048, cluster, groups, rs)
    run_grouped(ff, oracle, s, lengths, 7, cluster, groups)


@pytest.mark.parametrize("B,L,k", [(1, 1 << 20, 2048), (1, 300000, 1024), (4, 70000, 512), (64, 20000, 2048)])
def test_threshold_hint_is_exact_hit_or_miss(oracle, B, L, k):
    """A fitting guess takes the single-sweep path, a bad one falls back (status bit 8);
    both give the oracle's result, and the returned guess fits the next similar row."""
    from flash_float_jit_kernels_b200 import _lib, fast_topk_v3, new_threshold_hint
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(4242 + L)
    lengths = torch.full((B,), L, dtype=torch.int32)
    if B > 1:
        lengths[1] = L - 4097
        lengths[B - 1] = max(k + 5, L // 3)
    hint = new_threshold_hint(B, dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    missed = []
    for step in range(4):
        s = torch.randn((B, L), generator=g).to(torch.bfloat16).float()
        out = fast_topk_v3(s.to(dev), lengths.to(dev), k, status=status, threshold_hint=hint)
        torch.cuda.synchronize()
        st = int(status.item()); status.zero_()
        assert st & ~_lib.FF_STATUS_HINT_MISSED == 0
        missed.append(bool(st & _lib.FF_STATUS_HINT_MISSED))
        assert np.array_equal(out.cpu().numpy(), oracle.topk_c(s.numpy(), lengths.numpy(), k)), step
        assert not torch.isnan(hint).any()
    assert missed[0] is False           # no guess yet: nothing to miss
    if B == 1:   # the status word is shared by the batch: one row's miss sets it
        assert not all(missed[1:]), "guesses from the previous, similar row should mostly fit"
    # guesses that cannot fit: far too high (fewer than k pass), far too low (more than 4096 pass)
    for bad in (1e30, -1e30, float("inf"), float("-inf")):
        hint.fill_(bad)
        s = torch.randn((B, L), generator=g)
        out = fast_topk_v3(s.to(dev), lengths.to(dev), k, status=status, threshold_hint=hint)
        torch.cuda.synchronize()
        assert int(status.item()) == _lib.FF_STATUS_HINT_MISSED; status.zero_()
        assert np.array_equal(out.cpu().numpy(), oracle.topk_c(s.numpy(), lengths.numpy(), k)), bad


def test_threshold_hint_short_rows_and_special_values(oracle):
    from flash_float_jit_kernels_b200 import fast_topk_v3, new_threshold_hint
    dev = torch.device("cuda:0")
    B, L, k = 3, 9000, 512
    s = torch.randn((B, L), generator=torch.Generator().manual_seed(77))
    s[0, 100:200] = float("nan"); s[0, 300] = float("inf"); s[2, :] = 1.5       # NaN on top; an all-equal row
    lengths = torch.tensor([L, 400, L], dtype=torch.int32)                     # row 1 is shorter than k
    hint = new_threshold_hint(B, dev)
    for step in range(3):
        out = fast_topk_v3(s.to(dev), lengths.to(dev), k, threshold_hint=hint)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), oracle.topk_c(s.numpy(), lengths.numpy(), k)), step
    assert torch.isnan(hint[1])          # short row: no guess


@pytest.mark.parametrize("k", [1, 7, 2048])
def test_threshold_hint_edge_shapes(oracle, k):
    """Guesses with windows (row_starts), k = 1, rows barely longer than k, heavy ties and outliers."""
    from flash_float_jit_kernels_b200 import fast_topk_v3, new_threshold_hint
    dev = torch.device("cuda:0")
    B, L = 5, 6000
    g = torch.Generator().manual_seed(900 + k)
    lengths = torch.tensor([L - 100, max(k + 1, 50), 4097, L - 2048, 3000], dtype=torch.int32)
    starts = torch.tensor([100, 0, 3, 2048, 1], dtype=torch.int32)
    hint = new_threshold_hint(B, dev)
    for step in range(4):
        s = torch.randn((B, L), generator=g)
        s[2] = torch.round(s[2] * 2) / 2            # a few distinct values: ties far beyond 4096 per value
        s[3, ::97] += 50.0                          # far outliers
        if step == 2:
            s[4] = 0.25                             # constant row: the guess cannot separate anything
        out = fast_topk_v3(s.to(dev), lengths.to(dev), k, starts.to(dev), threshold_hint=hint)
        torch.cuda.synchronize()
        exp = oracle.topk_c(s.numpy(), lengths.numpy(), k, starts.numpy())
        assert np.array_equal(out.cpu().numpy(), exp), step
