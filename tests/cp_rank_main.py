"""One rank of the context-parallel top-k test (launched by torch.distributed.run).

``nccl``: real GPUs, the product path end to end.  ``gloo``: CPU ranks; the
two CUDA steps are replaced, in a test-only subclass, by the oracle's
statements so that the host logic (sharding, buffer layout, all-gather
plumbing, rank agreement) is exercised without a GPU.
"""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from flash_float_jit_kernels_b200.context_parallel import ContextParallelTopk, shard_bounds  # noqa: E402
from oracle import oracle  # noqa: E402


class OracleStepsPlan(ContextParallelTopk):
    """Test double: same buffers and exchange, CPU statements for the two kernels."""

    def _local(self, score_shard, lengths, shard_offset):
        v, g = oracle.cp_local(score_shard.numpy(), lengths.numpy(), self.k, shard_offset)
        self.send[0].copy_(torch.from_numpy(v.view(np.int32)))
        self.send[1].copy_(torch.from_numpy(g))

    def _merge(self, lengths):
        r = self.recv.numpy()
        out = oracle.cp_merge(r[:, 0].view(np.float32), r[:, 1], lengths.numpy(), self.k)
        self.out.copy_(torch.from_numpy(out))


def main():
    backend = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        device = torch.device("cuda", torch.cuda.current_device())
    else:
        device = torch.device("cpu")
    dist.init_process_group(backend, rank=rank, world_size=world)
    cases = [(1, 1 << 22, 2048, False), (2, 300001, 512, True)] if backend == "nccl" else \
            [(2, 50001, 128, True), (1, 4096, 64, False)]
    for B, L, k, ties in cases:
        g = torch.Generator().manual_seed(1234 + L)          # same full row on every rank
        s = torch.randn((B, L), generator=g)
        if ties:
            s = s.to(torch.bfloat16).float()
        lengths = torch.full((B,), L, dtype=torch.int32)
        if B > 1:
            lengths[1] = L - 777
        a, b = shard_bounds(L, world, rank)
        shard = s[:, a:b].contiguous().to(device)
        plan_cls = ContextParallelTopk if backend == "nccl" else OracleStepsPlan
        exp = oracle.topk_c(s.numpy(), lengths.numpy(), k)
        for exchange in (("p2p", "nccl") if backend == "nccl" else ("nccl",)):
            plan = plan_cls(B, k, device, exchange=exchange)
            assert plan.exchange == exchange
            for _ in range(3):                               # buffers are reused across calls
                out = plan(shard, lengths.to(device), a)
            if device.type == "cuda":
                torch.cuda.synchronize()
            assert np.array_equal(out.cpu().numpy(), exp), f"rank {rank}: mismatch B={B} L={L} k={k} {exchange}"
            plan.close()
        # every rank holds the same answer
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        assert all(torch.equal(gathered[0], t) for t in gathered)
    dist.barrier()
    if rank == 0:
        print("CP_OK", world, backend)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
