"""Host-side operator checks that need no GPU: argument errors and shard arithmetic."""
import pytest
import torch

from flash_float_jit_kernels_b200 import TopkArgumentError, fast_topk_v3, shard_bounds


def test_cpu_tensors_are_rejected_not_silently_computed():
    s = torch.randn(2, 64)
    l = torch.full((2,), 64, dtype=torch.int32)
    with pytest.raises(TopkArgumentError):
        fast_topk_v3(s, l, 8)


@pytest.mark.parametrize("bad_k", [0, -1, 2049, 3.5])
def test_bad_topk_raises_like_the_reference_assert(bad_k):
    s = torch.randn(2, 64)
    l = torch.full((2,), 64, dtype=torch.int32)
    with pytest.raises(AssertionError):          # reference: assert topk in (...)  topk_indexer.py:132
        fast_topk_v3(s, l, bad_k)
    with pytest.raises(ValueError):
        fast_topk_v3(s, l, bad_k)


def test_score_must_be_2d_float32():
    l = torch.full((2,), 64, dtype=torch.int32)
    with pytest.raises(TopkArgumentError):
        fast_topk_v3(torch.randn(2, 4, 16), l, 8)
    with pytest.raises(TopkArgumentError):
        fast_topk_v3(torch.randn(2, 64).double(), l, 8)


@pytest.mark.parametrize("L,P", [(4194304, 8), (8388608, 2), (1000003, 4), (17, 8), (5, 8), (4097, 3)])
def test_shard_bounds_partition_the_row(L, P):
    spans = [shard_bounds(L, P, r) for r in range(P)]
    assert spans[0][0] == 0 and spans[-1][1] == L
    for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
        assert a1 == b0 and a0 <= a1
    if L >= 4 * P:
        assert all(a % 4 == 0 for a, _ in spans)   # 16-byte aligned shard starts


def test_shard_bounds_rejects_bad_rank():
    with pytest.raises(TopkArgumentError):
        shard_bounds(100, 4, 4)


def test_reference_import_path_shim(monkeypatch):
    import sys
    from pathlib import Path
    import flash_float_jit_kernels_b200 as pkg
    monkeypatch.syspath_prepend(str(Path(pkg.__file__).parent / "compat"))
    sys.modules.pop("jit_kernel", None)
    sys.modules.pop("jit_kernel.topk_indexer", None)
    from jit_kernel.topk_indexer import fast_topk_v3 as shim
    assert shim is pkg.fast_topk_v3
    sys.modules.pop("jit_kernel", None)
    sys.modules.pop("jit_kernel.topk_indexer", None)


def test_cp_plan_status_surfaces_a_timeout_and_plan_is_a_context_manager():
    """The plan keeps one status word for all its steps; bit 2 (a bounded wait ran out) turns into
    an exception at the caller's sync point, other bits are returned and cleared."""
    from flash_float_jit_kernels_b200 import _lib
    from flash_float_jit_kernels_b200.context_parallel import ContextParallelTopk
    with ContextParallelTopk(2, 16, torch.device("cpu"), exchange="nccl") as plan:
        assert plan.check_status() == 0
        plan.status.fill_(_lib.FF_STATUS_HINT_MISSED)
        assert plan.check_status() == _lib.FF_STATUS_HINT_MISSED
        assert int(plan.status.item()) == 0, "read bits are cleared"
        plan.status.fill_(_lib.FF_STATUS_WAIT_TIMEOUT | _lib.FF_STATUS_HINT_MISSED)
        with pytest.raises(RuntimeError, match="re-synchronise"):
            plan.check_status()
        assert int(plan.status.item()) == 0
    assert plan._ex is None


def test_reference_arm_prints_one_complete_json_line():
    """``bench.py --impl reference`` needs no GPU: the CPU statement of the path, one JSON line with the
    keys of the bench contract, and the reason why the reference's own GPU kernel is not timed beside it."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    res = subprocess.run([sys.executable, str(root / "bench.py"), "--impl", "reference", "--steps", "3", "--warmup", "3"],
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "topk_us_per_call" and d["unit"] == "us" and d["higher_is_better"] is False
    assert d["value"] > 0 and d["n_gpus"] == 1 and d["steps"] == 3
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "unavailable" in d["reference_kernel_on_this_gpu"]
