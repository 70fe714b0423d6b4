"""The reference's own FFI symbol, ``fast_topk(score, indices, lengths, row_starts, has_row_starts)``
(``topk_indexer_radix.cu:1285-1290``, ``:1387``), exported by ``libff_topk_tvmffi.so``."""
import numpy as np
import pytest
import torch

tvm_ffi = pytest.importorskip("tvm_ffi")


@pytest.fixture(scope="module")
def module():
    from flash_float_jit_kernels_b200 import build
    path = build.tvmffi_lib_path()
    if not path.exists():
        build.build_tvmffi_module()
    return tvm_ffi.load_module(str(path))


def reference_wrapper_body(module, score, lengths, topk, row_starts=None):
    """What the reference's ``fast_topk_v3`` does once it holds its module
    (``jit_kernel/topk_indexer.py:137-151``, the TVM-FFI branch), statement for statement."""
    topk_indices = torch.full((score.size(0), topk), -1, dtype=torch.int32, device=score.device)
    rs = row_starts if row_starts is not None else torch.empty(0, dtype=torch.int32, device=score.device)
    module.fast_topk(score, topk_indices, lengths, rs, int(row_starts is not None))
    return topk_indices


def test_module_exports_the_reference_symbol_and_has_no_cpu_path(module):
    assert module.fast_topk is not None
    s = torch.randn(2, 64)
    l = torch.full((2,), 64, dtype=torch.int32)
    with pytest.raises(Exception, match="CUDA"):
        reference_wrapper_body(module, s, l, 8)


@pytest.mark.gpu
@pytest.mark.parametrize("B,L,topk,with_rs", [(1, 1 << 20, 2048, False), (3, 120000, 1024, True), (8, 65536, 512, False),
                                               (2, 16384, 2048, True)])
def test_reference_wrapper_runs_on_this_library(module, oracle, B, L, topk, with_rs):
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(B * 1000 + topk)
    s = (torch.rand((B, L), generator=g) * 255.0).to(torch.bfloat16).float()     # the reference's [0, 255] domain, with ties
    lengths = torch.full((B,), L - 2048 if with_rs else L, dtype=torch.int32)
    if B > 1:
        lengths[1] = 100                                                          # shorter than topk
    rs = torch.randint(0, 2048, (B,), generator=g, dtype=torch.int32) if with_rs else None
    for _ in range(2):                                                            # built-in scratch is reused
        out = reference_wrapper_body(module, s.to(dev), lengths.to(dev), topk, None if rs is None else rs.to(dev))
        torch.cuda.synchronize()
        exp = oracle.topk_c(s.numpy(), lengths.numpy(), topk, None if rs is None else rs.numpy())
        assert np.array_equal(out.cpu().numpy(), exp)


@pytest.mark.gpu
def test_reference_wrapper_uses_the_current_torch_stream(module, oracle):
    dev = torch.device("cuda:0")
    s = torch.randn((1, 300000), generator=torch.Generator().manual_seed(3))
    lengths = torch.tensor([300000], dtype=torch.int32)
    side = torch.cuda.Stream()
    sd, ld = s.to(dev), lengths.to(dev)
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        out = reference_wrapper_body(module, sd, ld, 512)
    side.synchronize()
    assert np.array_equal(out.cpu().numpy(), oracle.topk_c(s.numpy(), lengths.numpy(), 512))
