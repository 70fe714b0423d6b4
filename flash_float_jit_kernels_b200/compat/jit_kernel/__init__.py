"""Import-path shim: put ``flash_float_jit_kernels_b200/compat`` on ``sys.path``
and ``from jit_kernel.topk_indexer import fast_topk_v3`` resolves to the B200
implementation, so a caller of the reference (``jit_kernel/topk_indexer.py:109``)
switches without touching its imports.  Only the top-k indexer is provided."""
