"""bf16 / fp16 scores and 64-bit indices through the C ABI (``ff_topk_launch_typed``) against the
CPU oracle on the exact fp32 widening of the same values: bit-exact indices."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = {"bf16": torch.bfloat16, "f16": torch.float16}


@pytest.fixture(scope="module")
def ff():
    import flash_float_jit_kernels_b200 as pkg
    from flash_float_jit_kernels_b200 import _lib
    lib = _lib.load()
    assert lib.ff_topk_init(0) == 0
    yield pkg, lib
    lib.ff_topk_set_cluster_override(0)
    lib.ff_topk_set_groups_override(0)


def run_typed(ff, oracle, s16, lengths, k, rs=None, cluster=0, index_dtype=torch.int32, hint=None):
    pkg, lib = ff
    assert lib.ff_topk_set_cluster_override(cluster) == 0
    dev = torch.device("cuda:0")
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    before = lib.ff_topk_launch_count()
    out = pkg.fast_topk_v3(s16.to(dev), lengths.to(dev), k, None if rs is None else rs.to(dev), status=status,
                           index_dtype=index_dtype, threshold_hint=hint)
    torch.cuda.synchronize()
    assert lib.ff_topk_launch_count() == before + 1
    assert out.dtype == index_dtype
    bits = int(status.item())
    assert bits & ~8 == 0, f"device status {bits}"
    exp = oracle.topk_c(s16.float().numpy(), lengths.numpy(), k, None if rs is None else rs.numpy())
    got = out.cpu().numpy()
    assert np.array_equal(got.astype(np.int64), exp.astype(np.int64)), \
        f"mismatch at {np.argwhere(got != exp)[:5].tolist()}"
    return bits


@pytest.mark.parametrize("cluster", [0, 1, 2, 16])
def test_golden_vectors_in_their_own_16_bit_type(ff, golden, cluster):
    pkg, lib = ff
    lib.ff_topk_set_cluster_override(cluster)
    n = 0
    for name, c in golden.items():
        if c["bits16"] is None:
            continue
        s = torch.from_numpy(c["bits16"]).view(DTYPES[c["dtype"]]).cuda()
        rs = None if c["row_starts"] is None else torch.from_numpy(c["row_starts"]).cuda()
        out = pkg.fast_topk_v3(s, torch.from_numpy(c["lengths"]).cuda(), c["k"], rs)
        assert np.array_equal(out.cpu().numpy(), c["expected"]), f"{name} cluster={cluster}"
        n += 1
    assert n == 4


@pytest.mark.parametrize("tag", ["bf16", "f16"])
@pytest.mark.parametrize("L", [16384, 131072, 1048576])
def test_latency_sweep_rows_in_16_bit(ff, oracle, tag, L):
    s = torch.randn((1, L), generator=torch.Generator().manual_seed(L)).to(DTYPES[tag])   # heavy ties: few distinct values
    run_typed(ff, oracle, s, torch.tensor([L], dtype=torch.int32), 2048)


@pytest.mark.parametrize("tag", ["bf16", "f16"])
@pytest.mark.parametrize("cluster", [1, 4, 16])
def test_edge_lengths_and_misaligned_windows_in_16_bit(ff, oracle, tag, cluster):
    # 8 scores per 16-byte unit: window starts 1..7 elements into a unit, lengths around unit and k boundaries
    for L, k in ((2049, 2048), (4097, 512), (33, 32), (9, 8), (100003, 2048), (65543, 1)):
        s = torch.randn((4, L + 16), generator=torch.Generator().manual_seed(L * 7 + k)).to(DTYPES[tag])
        lengths = torch.tensor([L, max(0, L - 1), L // 2, L - 7], dtype=torch.int32)
        rs = torch.tensor([0, 1, 5, 7], dtype=torch.int32)
        run_typed(ff, oracle, s, lengths, k, rs, cluster=cluster)


@pytest.mark.parametrize("tag", ["bf16", "f16"])
def test_special_values_in_16_bit(ff, oracle, tag):
    dt = DTYPES[tag]
    x = torch.randn((3, 4096), generator=torch.Generator().manual_seed(9)).to(dt)
    x[0, ::7] = 0.0
    x[0, 3::7] = -0.0
    x[0, 5] = float("nan")
    x[0, 11] = float("inf")
    x[0, 12] = float("-inf")
    x[0, 13::97] = torch.tensor(6e-8 if tag == "f16" else 1e-40).to(dt)     # subnormals
    x[1, :] = 2.5                                                            # constant row: lowest indices win
    x[2, :] = torch.randint(0, 4, (4096,), generator=torch.Generator().manual_seed(10)).to(dt)
    for k in (64, 1000, 2048):
        run_typed(ff, oracle, x, torch.tensor([4096, 4096, 4000], dtype=torch.int32), k)


@pytest.mark.parametrize("tag", ["bf16", "f16"])
def test_ragged_decode_batch_in_16_bit(ff, oracle, tag):
    from flash_float_jit_kernels_b200 import workloads as W
    s, l, _ = W.lightning_indexer_logits(64, 131072, 4096, seed=2, device="cuda")
    run_typed(ff, oracle, s.to(DTYPES[tag]).cpu(), l.cpu(), 2048)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_int64_indices(ff, oracle, dtype):
    s = torch.randn((3, 70000), generator=torch.Generator().manual_seed(21)).to(dtype)
    lengths = torch.tensor([70000, 300, 0], dtype=torch.int32)            # a short row and an empty one: -1 padding in 64 bits
    run_typed(ff, oracle, s, lengths, 512, index_dtype=torch.int64)
    s = torch.randn((1, 1 << 20), generator=torch.Generator().manual_seed(22)).to(dtype)
    run_typed(ff, oracle, s, torch.tensor([1 << 20], dtype=torch.int32), 2048, index_dtype=torch.int64)


def test_threshold_guesses_with_bf16_scores(ff, oracle):
    from flash_float_jit_kernels_b200 import new_threshold_hint
    dev = torch.device("cuda:0")
    hint = new_threshold_hint(2, dev)
    base = torch.randn((2, 400000), generator=torch.Generator().manual_seed(31))
    seen = []
    for step in range(4):
        s = (base + 0.01 * torch.randn((2, 400000), generator=torch.Generator().manual_seed(32 + step))).to(torch.bfloat16)
        if step == 3:
            s = (s.float() * 4 + 10).to(torch.bfloat16)
        seen.append(run_typed(ff, oracle, s, torch.tensor([400000, 390000], dtype=torch.int32), 1024, hint=hint))
    assert seen[0] == 0 and seen[1] == 0 and seen[2] == 0
    assert seen[3] == 8, "the jump makes the guesses miss; the result stays exact"


def test_bad_dtype_and_index_width_are_rejected(ff):
    pkg, lib = ff
    dev = torch.device("cuda:0")
    s = torch.zeros((1, 64), device=dev)
    l = torch.full((1,), 64, dtype=torch.int32, device=dev)
    o = torch.empty((1, 8), dtype=torch.int32, device=dev)
    args = (s.stride(0), l.data_ptr(), None, o.data_ptr())
    assert lib.ff_topk_launch_typed(s.data_ptr(), 7, *args, 32, 1, 64, 8, None, None, None, 0, None, None) == -2
    assert lib.ff_topk_launch_typed(s.data_ptr(), 0, *args, 16, 1, 64, 8, None, None, None, 0, None, None) == -2
    with pytest.raises(pkg.TopkArgumentError):
        pkg.fast_topk_v3(s.double(), l, 8)
