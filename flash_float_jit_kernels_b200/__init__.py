"""B200-native exact radix top-k indexer.

Drop-in for the ``fast_topk_v3`` path of flash-float-jit-kernels
(``jit_kernel/topk_indexer.py:109``): same operator signature, hand-written
sm_100a CUDA behind a C ABI (``include/ff_topk.h``), no CPU fallback.
"""
from .topk_indexer import (  # noqa: F401
    TopkArgumentError,
    fast_topk_v3,
    fast_topk_transform_fused,
    fast_topk_transform_ragged_fused,
    new_threshold_hint,
)
from .context_parallel import (  # noqa: F401
    ContextParallelTopk,
    close_cached_plans,
    fast_topk_v3_cp,
    shard_bounds,
)

__all__ = [
    "TopkArgumentError",
    "fast_topk_v3",
    "fast_topk_transform_fused",
    "fast_topk_transform_ragged_fused",
    "new_threshold_hint",
    "fast_topk_v3_cp",
    "ContextParallelTopk",
    "close_cached_plans",
    "shard_bounds",
]
