"""ctypes binding of ``csrc/libff_topk.so`` (C ABI in ``include/ff_topk.h``).

There is no fallback: if the library is missing or a symbol is absent the
loader raises, so a GPU box can never silently run anything but the CUDA
kernels.
"""
from __future__ import annotations

import ctypes
import functools
from ctypes import c_char_p, c_int, c_int32, c_int64, c_size_t, c_void_p

from .build import lib_path

# name -> (restype, argtypes); mirrors include/ff_topk.h one to one
SIGNATURES = {
    "ff_topk_abi_version": (c_int32, []),
    "ff_last_error_string": (c_char_p, []),
    "ff_topk_launch_count": (c_int64, []),
    "ff_topk_init": (c_int, [c_int]),
    "ff_topk_set_cluster_override": (c_int, [c_int32]),
    "ff_topk_set_trace_buffer": (c_int, [c_void_p]),
    "ff_topk_set_groups_override": (c_int, [c_int32]),
    "ff_topk_set_self_seed": (c_int, [c_int32]),
    "ff_topk_set_programmatic_launch": (c_int, [c_int32]),
    "ff_topk_policy_cluster_size": (c_int32, [c_int32, c_int64, c_int32]),
    "ff_topk_policy_launch_shape": (c_int, [c_int32, c_int64, c_int32, c_int32, c_int32, ctypes.POINTER(c_int32)]),
    "ff_topk_workspace_bytes": (c_size_t, [c_int32, c_int64, c_int32]),
    "ff_topk_launch": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_int32,
         c_void_p, c_size_t, c_void_p, c_void_p],
    ),
    "ff_topk_launch_handover": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_int32,
         c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p],
    ),
    "ff_topk_launch_typed": (
        c_int,
        [c_void_p, c_int32, c_int64, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int64, c_int32,
         c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p],
    ),
    "ff_topk_launch_static": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_int32, c_void_p, c_void_p],
    ),
    "ff_topk_launch_hinted": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_int32,
         c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p],
    ),
    "ff_topk_transform_launch": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_int32, c_int32,
         c_void_p, c_int64, c_void_p, c_int32, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p],
    ),
    "ff_topk_cp_local": (
        c_int,
        [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_int32, c_int64,
         c_void_p, c_size_t, c_void_p, c_void_p],
    ),
    "ff_cp_exchange_create": (c_int, [c_int32, c_int32, c_int32, c_int32, ctypes.POINTER(c_void_p)]),
    "ff_cp_exchange_bytes": (c_int64, [c_void_p]),
    "ff_cp_exchange_base": (c_void_p, [c_void_p]),
    "ff_cp_exchange_ipc_handle": (c_int, [c_void_p, c_void_p]),
    "ff_cp_exchange_open_peers": (c_int, [c_void_p, c_void_p, c_int32]),
    "ff_cp_exchange_set_peer": (c_int, [c_void_p, c_int32, c_void_p]),
    "ff_cp_exchange_destroy": (c_int, [c_void_p]),
    "ff_topk_cp_send": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_size_t, c_void_p, c_void_p],
    ),
    "ff_topk_cp_recv_merge": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "ff_topk_cp_step": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_size_t, c_void_p,
         c_void_p],
    ),
    "ff_topk_cp_send_hinted": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_size_t,
         c_void_p, c_void_p],
    ),
    "ff_topk_cp_step_hinted": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
         c_size_t, c_void_p, c_void_p],
    ),
    "ff_topk_cp_step_emulated_ranks": (
        c_int,
        [c_int32, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_size_t, c_void_p, c_void_p],
    ),
    "ff_topk_cp_merge": (
        c_int,
        [c_void_p, c_void_p, c_int32, c_int64, c_void_p, c_void_p, c_int32, c_int32,
         c_void_p, c_size_t, c_void_p, c_void_p],
    ),
}

FF_EPILOGUE_INDEX = 0
FF_EPILOGUE_PAGE_TABLE = 1
FF_EPILOGUE_ADD_OFFSET = 2
FF_TOPK_MAX_K = 2048
FF_TOPK_HANDOVER_ROW_BYTES = 64 + 4096 * 8
FF_DTYPE_F32, FF_DTYPE_BF16, FF_DTYPE_F16 = 0, 1, 2
FF_STATUS_WAIT_TIMEOUT = 2
FF_STATUS_HINT_MISSED = 8
FF_STATUS_CP_SECOND_ROUND = 16
FF_STATUS_BOUNDS = 32
FF_STATUS_CP_SX_FALLBACK = 64
TRACE_SLOTS = 40


class LibraryMissingError(RuntimeError):
    pass


@functools.lru_cache(maxsize=None)
def load() -> ctypes.CDLL:
    """Load the CUDA library and attach the prototypes; raises if unavailable."""
    path = lib_path()
    if not path.exists():
        raise LibraryMissingError(
            f"{path} is missing: build it with `python -m flash_float_jit_kernels_b200.build` "
            "(there is no CPU or PyTorch fallback for the top-k indexer)"
        )
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise LibraryMissingError(f"{path} does not export {name}") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


@functools.lru_cache(maxsize=None)
def load_checked() -> ctypes.CDLL:
    """The bounds-checked build of the same library (``build.build_checked_library``), for debugging
    and for the test that runs the golden vectors through it; same prototypes."""
    from .build import checked_lib_path
    path = checked_lib_path()
    if not path.exists():
        raise LibraryMissingError(f"{path} is missing: build it with "
                                  "`python -m flash_float_jit_kernels_b200.build --checked`")
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


def check(rc: int, what: str) -> None:
    """Turn a non-zero return code into the exception the wrapper documents."""
    if rc == 0:
        return
    msg = load().ff_last_error_string().decode("utf-8", "replace")
    if rc < 0:
        raise ValueError(f"{what}: {msg} (code {rc})")
    raise RuntimeError(f"{what}: CUDA error {rc}: {msg}")
