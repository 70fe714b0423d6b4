"""Selects launched with programmatic stream serialization (the default) read what the kernel before
them on the stream wrote, leave their scratch clean for the next one, and give the same result as in
plain stream order: chains of dependent launches, eager and replayed from a CUDA graph."""
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
    lib.ff_topk_set_programmatic_launch(-1)


def _variants(B, L, n, seed):
    g = torch.Generator().manual_seed(seed)
    s = torch.randn((n, B, L), generator=g).to(torch.bfloat16).float()
    lengths = torch.randint(L // 2, L + 1, (B,), generator=g, dtype=torch.int32)
    return s, lengths


@pytest.mark.parametrize("B,L,k", [(1, 1 << 20, 2048), (2, 262144, 1024), (64, 32768, 2048), (4, 16384, 512)])
@pytest.mark.parametrize("on", [1, 0])
def test_chain_in_a_graph(ff, oracle, B, L, k, on):
    """Every step of the chain overwrites the ONE score buffer (a copy kernel) and selects from it
    right away; a select that started before the copy was done, or before the select in front of it
    had cleaned the row scratch, would give a wrong row."""
    pkg, lib = ff
    lib.ff_topk_set_programmatic_launch(on)
    dev = torch.device("cuda:0")
    n = 6
    s, lengths = _variants(B, L, n, seed=B * 1000 + k)
    src = s.to(dev)
    ld = lengths.to(dev)
    buf = torch.empty((B, L), dtype=torch.float32, device=dev)
    outs = torch.full((n, B, k), -7, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    hint = pkg.new_threshold_hint(B, dev)

    def chain(with_hint):
        for i in range(n):
            buf.copy_(src[i])
            pkg.fast_topk_v3(buf, ld, k, out=outs[i], status=status, threshold_hint=hint if with_hint else None)

    exp = [oracle.topk_c(s[i].numpy(), lengths.numpy(), k) for i in range(n)]
    for with_hint in (False, True):
        chain(with_hint)                                   # eager
        torch.cuda.synchronize()
        for i in range(n):
            assert np.array_equal(outs[i].cpu().numpy(), exp[i]), f"eager step {i}"
        outs.fill_(-7)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                chain(with_hint)
            for _ in range(3):
                graph.replay()
            side.synchronize()
        for i in range(n):
            assert np.array_equal(outs[i].cpu().numpy(), exp[i]), f"graph step {i}"
        assert int(status.item()) & ~8 == 0                # a guess may miss; nothing else may be set


def test_selects_back_to_back_share_the_row_scratch(ff, oracle):
    """Split rows (global scratch, cooperative launch) one directly behind the other, no kernel between."""
    pkg, lib = ff
    lib.ff_topk_set_programmatic_launch(1)
    dev = torch.device("cuda:0")
    n, L, k = 8, 1 << 20, 2048
    s, _ = _variants(1, L, n, seed=5)
    src = s.to(dev)
    ld = torch.tensor([L - 3], dtype=torch.int32, device=dev)
    outs = torch.full((n, 1, k), -7, dtype=torch.int32, device=dev)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        pkg.fast_topk_v3(src[0], ld, k, out=outs[0])
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(n):
                pkg.fast_topk_v3(src[i], ld, k, out=outs[i])
        for _ in range(5):
            graph.replay()
        side.synchronize()
    lengths = np.array([L - 3], dtype=np.int32)
    for i in range(n):
        assert np.array_equal(outs[i].cpu().numpy(), oracle.topk_c(s[i].numpy(), lengths, k)), f"step {i}"
