"""The C-ABI library loads, exports every declared symbol, and rejects bad arguments before touching a GPU."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    from flash_float_jit_kernels_b200 import _lib, build
    build.build_library()
    return _lib.load()


def declared_functions():
    text = (ROOT / "include" / "ff_topk.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ff_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("ff_topk_launch", "ff_topk_transform_launch", "ff_topk_cp_local", "ff_topk_cp_merge",
                 "ff_topk_init", "ff_topk_workspace_bytes", "ff_last_error_string"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    from flash_float_jit_kernels_b200 import _lib
    raw = ctypes.CDLL(str(_lib.lib_path()))
    for name in declared_functions():
        assert hasattr(raw, name), f"{name} declared in include/ff_topk.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes prototype"


def test_abi_version(lib):
    assert lib.ff_topk_abi_version() >= 1


def test_argument_errors_need_no_gpu(lib):
    # validation happens before any CUDA call, so this runs on a CPU-only box
    assert lib.ff_topk_launch(None, 0, None, None, None, 1, 16, 0, None, 0, None, None) == -1
    assert b"k must be" in lib.ff_last_error_string()
    assert lib.ff_topk_launch(None, 0, None, None, None, 1, 16, 4096, None, 0, None, None) == -1
    assert lib.ff_topk_launch(None, 0, None, None, None, -1, 16, 8, None, 0, None, None) == -2
    assert lib.ff_topk_launch(None, 0, None, None, None, 1, 16, 8, None, 0, None, None) == -3
    assert lib.ff_topk_launch(None, 0, None, None, None, 1, 2**31, 8, None, 0, None, None) == -6
    assert lib.ff_topk_set_cluster_override(3) == -5
    assert lib.ff_topk_set_cluster_override(0) == 0
    assert lib.ff_topk_cp_merge(None, None, 0, 0, None, None, 1, 8, None, 0, None, None) == -2
    # B == 0 is a no-op that succeeds without a device
    assert lib.ff_topk_launch(None, 0, None, None, None, 0, 16, 8, None, 0, None, None) == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from flash_float_jit_kernels_b200 import _lib
    _lib.load.cache_clear()
    monkeypatch.setattr(_lib, "lib_path", lambda: tmp_path / "libff_topk.so")
    with pytest.raises(_lib.LibraryMissingError):
        _lib.load()
    monkeypatch.undo()
    _lib.load.cache_clear()
    _lib.load()
