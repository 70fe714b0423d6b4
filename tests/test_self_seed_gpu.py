"""Rows split over clusters make their own threshold guess when the caller gives none: exact on rows
where the guess fits (i.i.d.-like) and on rows where it cannot (trends, sorted rows, all winners in
one chunk, constant rows, heavy ties), and a miss of the row's own guess is not reported."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ff():
    import flash_float_jit_kernels_b200 as pkg
    from flash_float_jit_kernels_b200 import _lib
    lib = _lib.load()
    assert lib.ff_topk_init(0) == 0
    yield pkg, lib
    lib.ff_topk_set_self_seed(-1)
    lib.ff_topk_set_cluster_override(0)
    lib.ff_topk_set_groups_override(0)


def _run(ff, oracle, s, lengths, k, expect_seeded=None):
    """Runs one launch with the stage trace on; returns whether any CTA stamped the own-guess stage."""
    pkg, lib = ff
    dev = torch.device("cuda:0")
    from flash_float_jit_kernels_b200 import _lib
    trace = torch.zeros((s.shape[0] * 1024, _lib.TRACE_SLOTS), dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    sd, ld = s.to(dev), lengths.to(dev)
    lib.ff_topk_set_trace_buffer(trace.data_ptr())
    try:
        out = pkg.fast_topk_v3(sd, ld, k, status=status)
        torch.cuda.synchronize()
    finally:
        lib.ff_topk_set_trace_buffer(None)
    assert int(status.item()) == 0, f"status {int(status.item())}: a miss of the row's own guess must not be reported"
    exp = oracle.topk_c(s.numpy(), lengths.numpy(), k)
    assert np.array_equal(out.cpu().numpy(), exp)
    seeded = bool((trace[:, 21] != 0).any())
    if expect_seeded is not None:
        assert seeded == expect_seeded
    # a second launch right away: the scratch was left clean whatever path the first one took
    out2 = pkg.fast_topk_v3(sd, ld, k, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and np.array_equal(out2.cpu().numpy(), exp)
    return seeded


@pytest.mark.parametrize("L,k", [(1 << 20, 2048), (1 << 20, 512), (262144, 2048), (1 << 22, 2048), (1000003, 1024),
                                 (1 << 24, 2048), ((1 << 24) - 4099, 2048)])   # the last two: guessed from two tiles
def test_own_guess_on_exchangeable_rows(ff, oracle, L, k):
    pkg, lib = ff
    lib.ff_topk_set_self_seed(1)
    g = torch.Generator().manual_seed(L + k)
    s = torch.randn((1, L), generator=g)
    _run(ff, oracle, s, torch.tensor([L], dtype=torch.int32), k, expect_seeded=True)
    s = s.to(torch.bfloat16).float()                       # heavy ties
    _run(ff, oracle, s, torch.tensor([L - 777], dtype=torch.int32), k, expect_seeded=True)


@pytest.mark.parametrize("shape", ["ascending", "descending", "trend", "one_chunk", "constant", "two_values", "spike_tail", "nan_inf"])
def test_own_guess_that_cannot_fit_falls_back(ff, oracle, shape):
    pkg, lib = ff
    lib.ff_topk_set_self_seed(1)
    L, k = 1 << 20, 2048
    g = torch.Generator().manual_seed(17)
    x = torch.randn((1, L), generator=g)
    if shape == "ascending":
        s = torch.sort(x, dim=1).values
    elif shape == "descending":
        s = torch.sort(x, dim=1, descending=True).values
    elif shape == "trend":
        s = x + torch.linspace(0.0, 12.0, L).unsqueeze(0)
    elif shape == "one_chunk":
        s = x.clone()
        s[0, 500000:503000] += 20.0                         # every winner sits in one CTA's chunk
    elif shape == "constant":
        s = torch.full((1, L), -3.25)
    elif shape == "two_values":
        s = (x > 2.0).float()                               # 2 % ones: far more than 4096 tie at the top
    elif shape == "spike_tail":
        s = x.clone()
        s[0, ::4096] = 1e30                                 # every CTA sees huge maxima that say nothing about rank 2048
    else:
        s = x.clone()
        s[0, ::1000] = float("nan")
        s[0, 1::1000] = float("inf")
        s[0, 2::1000] = float("-inf")
    _run(ff, oracle, s, torch.tensor([L], dtype=torch.int32), k)


def test_own_guess_can_be_switched_off_and_batches_of_long_rows_work(ff, oracle):
    pkg, lib = ff
    g = torch.Generator().manual_seed(5)
    s = torch.randn((2, 1 << 20), generator=g).to(torch.bfloat16).float()
    lengths = torch.tensor([1 << 20, 900001], dtype=torch.int32)
    lib.ff_topk_set_self_seed(0)
    assert _run(ff, oracle, s, lengths, 2048) is False
    lib.ff_topk_set_self_seed(1)
    assert _run(ff, oracle, s, lengths, 2048) is True
    # short rows are not split over clusters: nothing to seed
    s = torch.randn((3, 30000), generator=g)
    assert _run(ff, oracle, s, torch.tensor([30000, 20000, 100], dtype=torch.int32), 512) is False
