"""Drop-in for ``jit_kernel/topk_indexer.py`` of the reference: same public name
and signature (``fast_topk_v3(score, lengths, topk, row_starts=None)``)."""
from flash_float_jit_kernels_b200.topk_indexer import (  # noqa: F401
    fast_topk_transform_fused,
    fast_topk_transform_ragged_fused,
    fast_topk_v3,
)

__all__ = ["fast_topk_v3", "fast_topk_transform_fused", "fast_topk_transform_ragged_fused"]
