"""The allocation-free entry point against the ordinary one.

``ff_topk_launch_static`` is for hosts that may not allocate device memory (a
plugin inside a runtime that owns all buffers, a frozen memory pool, a place
where ``cudaMalloc`` would stall the device): it uses scratch compiled into the
library instead of a caller workspace.  This file is collected last on purpose,
so a run that stops at the first failure has already run every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, fn_name, s, lengths, out, k, ws=None):
    stream = torch.cuda.current_stream().cuda_stream
    if fn_name == "static":
        return lib.ff_topk_launch_static(s.data_ptr(), s.stride(0), lengths.data_ptr(), None, out.data_ptr(),
                                         s.size(0), s.size(1), k, None, stream)
    return lib.ff_topk_launch(s.data_ptr(), s.stride(0), lengths.data_ptr(), None, out.data_ptr(),
                              s.size(0), s.size(1), k, None if ws is None else ws.data_ptr(),
                              0 if ws is None else ws.numel(), None, stream)


def _free_bytes():
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row(oracle):
    from flash_float_jit_kernels_b200 import _lib
    assert torch.cuda.is_available()
    lib = _lib.load()
    lib.ff_topk_set_cluster_override(0)
    lib.ff_topk_set_groups_override(0)
    dev = torch.device("cuda:0")
    B, L, k = 2, 1 << 20, 2048                      # long rows: both entry points split them over clusters
    g = torch.Generator(device=dev)
    g.manual_seed(77)
    lengths = torch.tensor([L, L - 4321], dtype=torch.int32, device=dev)
    need = int(lib.ff_topk_workspace_bytes(B, L, k))
    assert need > 0, "this shape is meant to exercise the scratch-using kernel path"
    ws = torch.zeros(need, dtype=torch.uint8, device=dev)
    for call in range(2):                           # two calls in a row: the scratch is shared and reused
        s = torch.randn((B, L), generator=g, device=dev).to(torch.bfloat16).float()
        ref = torch.full((B, k), -7, dtype=torch.int32, device=dev)
        got = torch.full((B, k), -9, dtype=torch.int32, device=dev)
        assert _call(lib, "workspace", s, lengths, ref, k, ws) == 0
        free_before = _free_bytes()
        assert _call(lib, "static", s, lengths, got, k) == 0, lib.ff_last_error_string()
        # the driver reports free device memory for the whole GPU: had the call allocated anything
        # (cudaMalloc rounds up to at least 2 MiB here), the figure would have dropped
        assert _free_bytes() == free_before, f"call {call}: free device memory changed across the call"
        assert torch.equal(got, ref), f"call {call}: entry points disagree"   # integer indices: exact
        exp = oracle.topk_c(s.cpu().numpy(), lengths.cpu().numpy(), k)         # and both agree with the CPU oracle
        assert np.array_equal(got.cpu().numpy(), exp), f"call {call}: disagrees with the oracle"
    # short rows take the scratch-free kernel path; the entry point must still agree
    s = torch.randn((3, 5000), generator=g, device=dev)
    l3 = torch.tensor([5000, 17, 4000], dtype=torch.int32, device=dev)
    ref = torch.empty((3, 64), dtype=torch.int32, device=dev)
    got = torch.empty((3, 64), dtype=torch.int32, device=dev)
    assert _call(lib, "workspace", s, l3, ref, 64) == 0
    assert _call(lib, "static", s, l3, got, 64) == 0
    torch.cuda.synchronize()
    assert torch.equal(got, ref)
    assert np.array_equal(got.cpu().numpy(), oracle.topk_c(s.cpu().numpy(), l3.cpu().numpy(), 64))


def test_static_scratch_entry_rejects_more_rows_than_its_scratch_holds():
    from flash_float_jit_kernels_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    s = torch.zeros((5, 4096), device=dev)
    lengths = torch.full((5,), 4096, dtype=torch.int32, device=dev)
    out = torch.empty((5, 8), dtype=torch.int32, device=dev)
    assert _call(lib, "static", s, lengths, out, 8) == -6          # FF_ERR_TOO_LARGE
    assert b"FF_TOPK_STATIC_MAX_ROWS" in lib.ff_last_error_string()
