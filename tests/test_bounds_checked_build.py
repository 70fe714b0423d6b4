"""The build with -DFF_BOUNDS_CHECK (range-checked indices that set a status bit instead of touching
memory) run on the golden vectors and on the shapes whose work arrays fill up: it must give the
same exact results and never raise FF_STATUS_BOUNDS."""
import numpy as np
import pytest
import torch


def test_checked_library_exports_the_same_symbols():
    from flash_float_jit_kernels_b200 import _lib, build
    build.build_checked_library()
    lib = _lib.load_checked()
    for name in _lib.SIGNATURES:
        assert hasattr(lib, name), name


def _launch(lib, s, lengths, k, rs=None, hint=None):
    dev = s.device
    B, L = s.shape
    out = torch.empty((B, k), dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    need = int(lib.ff_topk_workspace_bytes(B, L, k))
    ws = torch.zeros(max(need, 256), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    if hint is None:
        rc = lib.ff_topk_launch(s.data_ptr(), s.stride(0), lengths.data_ptr(), None if rs is None else rs.data_ptr(),
                                out.data_ptr(), B, L, k, ws.data_ptr() if need else None, need, status.data_ptr(), stream)
    else:
        rc = lib.ff_topk_launch_hinted(s.data_ptr(), s.stride(0), lengths.data_ptr(), None, out.data_ptr(), B, L, k,
                                       hint.data_ptr(), hint.data_ptr(), ws.data_ptr() if need else None, need,
                                       status.data_ptr(), stream)
    assert rc == 0, lib.ff_last_error_string()
    torch.cuda.synchronize()
    return out, int(status.item())


@pytest.mark.gpu
def test_golden_vectors_through_the_checked_build(golden):
    from flash_float_jit_kernels_b200 import _lib
    lib = _lib.load_checked()
    assert lib.ff_topk_init(0) == 0
    for cluster in (0, 1, 4, 16):
        assert lib.ff_topk_set_cluster_override(cluster) == 0
        for name, c in golden.items():
            s = torch.from_numpy(c["score"]).cuda()
            l = torch.from_numpy(c["lengths"]).cuda()
            rs = None if c["row_starts"] is None else torch.from_numpy(c["row_starts"]).cuda()
            out, status = _launch(lib, s, l, c["k"], rs)
            assert status & _lib.FF_STATUS_BOUNDS == 0, f"{name} cluster={cluster}: status {status:#x}"
            assert np.array_equal(out.cpu().numpy(), c["expected"]), f"{name} cluster={cluster}"
    lib.ff_topk_set_cluster_override(0)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", ["ties_1m", "constant", "few_distinct", "ragged_b64", "hinted"])
def test_full_work_arrays_through_the_checked_build(oracle, shape):
    from flash_float_jit_kernels_b200 import _lib, new_threshold_hint, workloads as W
    lib = _lib.load_checked()
    dev = torch.device("cuda:0")
    hint = None
    if shape == "ties_1m":
        s, l, _ = W.gaussian_bf16_ties(1, 1 << 20, seed=3)
        k = 2048
    elif shape == "constant":          # one bucket holds every survivor: the case that once overran the unit queue
        s, l, k = torch.full((2, 300000), 2.5), torch.tensor([300000, 299999], dtype=torch.int32), 2048
    elif shape == "few_distinct":
        g = torch.Generator().manual_seed(4)
        s = torch.randint(0, 3, (2, 200000), generator=g).float()
        l, k = torch.tensor([200000, 150000], dtype=torch.int32), 1024
    elif shape == "ragged_b64":
        s, l, _ = W.lightning_indexer_logits(64, 65536, 4096, seed=6, device="cuda")
        s, l, k = s.cpu(), l.cpu(), 2048
    else:
        s, l, _ = W.gaussian_bf16_ties(2, 400000, seed=8)
        k = 1024
        hint = new_threshold_hint(2, dev)
    sd, ld = s.to(dev), l.to(dev)
    exp = oracle.topk_c(s.numpy(), l.numpy(), k)
    for _ in range(2 if hint is not None else 1):
        out, status = _launch(lib, sd, ld, k, hint=hint)
        assert status & _lib.FF_STATUS_BOUNDS == 0, f"status {status:#x}"
        assert np.array_equal(out.cpu().numpy(), exp)
