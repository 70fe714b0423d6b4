"""Context-parallel mode on GPUs: shards emulated on one device, and real ranks over NCCL when >= 2 GPUs."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("P", [1, 2, 4, 8])
@pytest.mark.parametrize("ties", [False, True])
def test_sharded_select_and_merge_on_one_device(oracle, P, ties):
    """All P shards run back to back on one GPU through the same C entry points the ranks use."""
    from flash_float_jit_kernels_b200 import _lib, shard_bounds
    lib = _lib.load()
    lib.ff_topk_set_cluster_override(0)
    dev = torch.device("cuda:0")
    B, L, k = 2, 1 << 20, 2048
    g = torch.Generator().manual_seed(100 + P)
    s = torch.randn((B, L), generator=g)
    if ties:
        s = s.to(torch.bfloat16).float()
    lengths = torch.tensor([L, L - 12345], dtype=torch.int32)
    sd, ld = s.to(dev), lengths.to(dev)
    recv = torch.empty((P, 2, B, k), dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    for r in range(P):
        a, b = shard_bounds(L, P, r)
        shard = sd[:, a:b]
        rc = lib.ff_topk_cp_local(shard.data_ptr(), shard.stride(0), ld.data_ptr(), recv[r, 1].data_ptr(),
                                  recv[r, 0].data_ptr(), B, b - a, k, a, None, 0, None, stream)
        assert rc == 0
    out = torch.empty((B, k), dtype=torch.int32, device=dev)
    rc = lib.ff_topk_cp_merge(recv[0, 0].data_ptr(), recv[0, 1].data_ptr(), P, 2 * B * k, ld.data_ptr(),
                              out.data_ptr(), B, k, None, 0, None, stream)
    assert rc == 0
    torch.cuda.synchronize()
    # the shard-local candidates themselves match the oracle's statement of step 1
    a, b = shard_bounds(L, P, P - 1)
    v, gi = oracle.cp_local(np.ascontiguousarray(s[:, a:b].numpy()), lengths.numpy(), k, a)
    assert np.array_equal(recv[P - 1, 1].cpu().numpy(), gi)
    assert np.array_equal(recv[P - 1, 0].cpu().numpy().view(np.float32), v)
    assert np.array_equal(out.cpu().numpy(), oracle.topk_c(s.numpy(), lengths.numpy(), k))


def test_short_global_rows_in_cp_mode(oracle):
    from flash_float_jit_kernels_b200 import _lib, shard_bounds
    lib = _lib.load()
    dev = torch.device("cuda:0")
    B, L, k, P = 3, 40000, 512, 4
    s = torch.randn((B, L), generator=torch.Generator().manual_seed(5))
    lengths = torch.tensor([300, 10001, 512], dtype=torch.int32)   # row 0/2: <= k; row 1 ends inside shard 1
    sd, ld = s.to(dev), lengths.to(dev)
    recv = torch.empty((P, 2, B, k), dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    for r in range(P):
        a, b = shard_bounds(L, P, r)
        shard = sd[:, a:b]
        assert lib.ff_topk_cp_local(shard.data_ptr(), shard.stride(0), ld.data_ptr(), recv[r, 1].data_ptr(),
                                    recv[r, 0].data_ptr(), B, b - a, k, a, None, 0, None, stream) == 0
    out = torch.empty((B, k), dtype=torch.int32, device=dev)
    assert lib.ff_topk_cp_merge(recv[0, 0].data_ptr(), recv[0, 1].data_ptr(), P, 2 * B * k, ld.data_ptr(),
                                out.data_ptr(), B, k, None, 0, None, stream) == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), oracle.topk_c(s.numpy(), lengths.numpy(), k))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_real_ranks_over_nccl():
    n = min(torch.cuda.device_count(), 8)
    n = 1 << (n.bit_length() - 1)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29531", str(ROOT / "tests" / "cp_rank_main.py"), "nccl"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "CP_OK" in res.stdout
