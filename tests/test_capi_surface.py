"""The C-ABI library: it loads, exports every function the public header declares, and rejects bad
arguments before touching the device (so these run without a GPU)."""
from __future__ import annotations

import ctypes
import pathlib
import re

import pytest

from nibble_b200 import _native

HEADER = pathlib.Path(__file__).resolve().parent.parent / "include" / "w4a16_b200.h"


def declared_functions() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(w4a16_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_table_agree():
    assert declared_functions() == sorted(_native.C_API)


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(_native.CORE_LIB))
    for name in declared_functions():
        assert hasattr(lib, name), name


def test_version_and_status_strings():
    lib = _native.core()
    assert lib.w4a16_abi_version() == 2
    assert _native.status_string(0) == "ok"
    for code in range(-8, 0):
        assert _native.status_string(code) not in ("ok", "unknown status")
    assert _native.status_string(-99) == "unknown status"


def test_argument_validation_happens_before_any_launch():
    lib = _native.core()
    before = lib.w4a16_launch_count()
    f = lib.w4a16_linear_f16
    one = ctypes.c_void_p(16)
    assert f(one, one, one, one, 1, 8, 127, 128, None, 0, 0, None) == -2   # odd K
    assert f(one, one, one, one, 1, 8, 192, 128, None, 0, 0, None) == -2   # K % group
    assert f(one, one, one, one, -1, 8, 128, 128, None, 0, 0, None) == -2  # negative M
    assert f(one, one, one, one, 1, 8, 128, 0, None, 0, 0, None) == -3     # group <= 0
    assert f(one, one, one, one, 1, 8, 126, 63, None, 0, 0, None) == -3    # odd group
    assert f(None, one, one, one, 1, 8, 128, 128, None, 0, 0, None) == -1  # NULL x
    assert f(one, one, one, None, 1, 8, 128, 128, None, 0, 0, None) == -1  # NULL y
    assert f(None, None, None, None, 0, 8, 128, 128, None, 0, 0, None) == 0  # empty: ok, nothing runs
    assert f(None, None, None, None, 4, 0, 128, 128, None, 0, 0, None) == 0
    d = lib.w4a16_dequantize_f16
    assert d(one, one, one, 8, 128, 48, None) == -3    # group not a multiple of 32
    assert d(one, one, one, 8, 96, 64, None) == -2     # K % group
    assert d(ctypes.c_void_p(8), one, one, 8, 128, 128, None) == -4  # packed not 16-byte aligned
    assert d(None, one, one, 8, 128, 128, None) == -1
    assert d(None, None, None, 0, 128, 128, None) == 0
    cfg = _native.LinearConfig(1, 8, 1, 1, 0)
    g = lib.w4a16_linear_f16_config
    assert g(one, one, one, one, 1, 8, 128, 64, None, 0, 0, ctypes.byref(cfg), None) == -6  # fast path n/a
    assert g(one, one, one, one, 1, 8, 128, 128, None, 0, 0, None, None) == -1
    assert lib.w4a16_launch_count() == before


def test_workspace_size_query():
    lib = _native.core()
    assert lib.w4a16_linear_workspace_bytes(0, 8, 128) == 0
    assert lib.w4a16_linear_workspace_bytes(1, 8, 100) == 0
    # a tall-K, few-rows problem asks for split-K scratch; a wide one does not
    assert lib.w4a16_linear_workspace_bytes(1, 1024, 8192) > 0
    assert lib.w4a16_linear_workspace_bytes(1, 32000, 2048) == 0
    # prefill-sized batches run the tcgen05 GEMM, which has no scratch -- unless a flag keeps them off it
    assert lib.w4a16_linear_workspace_bytes(512, 8192, 8192) == 0
    assert lib.w4a16_linear_workspace_bytes_flags(512, 8192, 8192, 0) == 0
    assert lib.w4a16_linear_workspace_bytes_flags(512, 8192, 8192, _native.FLAG_NO_TCGEN05) > 0
    assert lib.w4a16_linear_workspace_bytes_flags(512, 8192, 8192, _native.FLAG_OUTPUT_F32) > 0
    assert lib.w4a16_linear_workspace_bytes_flags(1, 1024, 8192, _native.FLAG_FORCE_GENERIC) == 0
    assert lib.w4a16_linear_workspace_bytes_flags(16, 8192, 8192, 0) == lib.w4a16_linear_workspace_bytes(16, 8192, 8192) > 1 << 20
    # 17..64 rows: large layers go to the GEMM as well (no scratch), small ones stay on the streaming kernel
    # (the GEMM wants scratch of its own only for layers of few tiles, to share their K between CTAs: 64 tiles here)
    assert 0 < lib.w4a16_linear_workspace_bytes(32, 8192, 8192) < 3 << 20
    assert lib.w4a16_linear_workspace_bytes_flags(32, 8192, 8192, _native.FLAG_NO_TCGEN05) > 4 << 20
    assert lib.w4a16_linear_workspace_bytes(32, 1024, 8192) > 0
    assert lib.w4a16_linear_workspace_bytes_flags(8, 28672, 8192, _native.FLAG_FORCE_TCGEN05) == 0
    assert lib.w4a16_linear_workspace_bytes_flags(8, 1024, 8192, _native.FLAG_FORCE_TCGEN05) == 256 * 1024 + 4 * 8 * 1024 * 4
    assert lib.w4a16_linear_workspace_bytes_flags(128, 256, 2048, _native.FLAG_FORCE_TCGEN05) == 0    # K below 4096 is not shared


def test_missing_library_is_an_error(monkeypatch, tmp_path):
    monkeypatch.setattr(_native, "CORE_LIB", tmp_path / "absent.so")
    _native.core.cache_clear()
    try:
        with pytest.raises(RuntimeError, match="not built"):
            _native.core()
    finally:
        monkeypatch.undo()
        _native.core.cache_clear()
