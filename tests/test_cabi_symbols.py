"""The C-ABI library loads, exports every function include/b200k.h declares, and the Python binding
types each of them.  Also exercises the entry points that return before touching a device."""
import ctypes
import re
from pathlib import Path

import pytest

from triton_tenstorrent_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "b200k.h").read_text()


def declared_functions():
    # strip comments, then take every identifier b200k_* followed by "(" at declaration level
    text = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    names = re.findall(r"\b(b200k_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_expected_entry_points():
    names = declared_functions()
    for must in ("b200k_add_f32", "b200k_sin_f32", "b200k_matmul_bf16", "b200k_attn_fwd_bf16", "b200k_launch",
                 "b200k_device_props", "b200k_block_range", "b200k_last_error", "b200k_version"):
        assert must in names


@pytest.mark.parametrize("name", declared_functions())
def test_symbol_exported_and_bound(name):
    lib = _lib.load()
    assert hasattr(lib, name), f"{name} is declared in include/b200k.h but not exported by {_lib.LIB_PATH.name}"
    assert name in _lib.SIGNATURES, f"{name} has no ctypes signature in _lib.SIGNATURES"


def test_binding_has_no_extra_symbols():
    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_version_and_block_range():
    lib = _lib.load()
    assert lib.b200k_version() >= 100
    s, e = ctypes.c_int64(), ctypes.c_int64()
    covered = []
    for w in range(5):
        assert lib.b200k_block_range(97, 5, w, ctypes.byref(s), ctypes.byref(e)) == _lib.OK
        covered.extend(range(s.value, e.value))
    assert covered == list(range(97))
    assert lib.b200k_block_range(10, 0, 0, ctypes.byref(s), ctypes.byref(e)) == _lib.ERR_INVALID_ARG
    assert "block_range" in _lib.last_error()


def test_argument_errors_before_any_device_work():
    lib = _lib.load()
    assert lib.b200k_add_f32(None, None, None, -1, 1024, None) == _lib.ERR_INVALID_ARG
    assert "n must be >= 0" in _lib.last_error()
    assert lib.b200k_sin_f32(None, None, 8, 0, None) == _lib.ERR_INVALID_ARG
    assert lib.b200k_add_f32(None, None, None, 8, 1024, None) == _lib.ERR_INVALID_ARG  # null pointers
    assert lib.b200k_matmul_bf16(None, None, None, 0, 8, 8, 8, 8, 8, None, 0, 0, 0, 0, None) == _lib.ERR_INVALID_ARG
    assert lib.b200k_matmul_bf16(16, 16, 16, 8, 8, 8, 12, 8, 8, None, 0, 0, 0, 0, None) == _lib.ERR_INVALID_ARG
    assert "multiples of 8" in _lib.last_error()
    assert lib.b200k_attn_fwd_bf16(16, 16, 16, 16, 16, 1, 1, 128, 48, 0, 0.1, None) == _lib.ERR_UNSUPPORTED   # HEAD_DIM 48
    assert lib.b200k_attn_supported(128, 4096) == 1 and lib.b200k_attn_supported(64, 256) == 1
    assert lib.b200k_attn_supported(16, 128) == 1 and lib.b200k_attn_supported(256, 4096) == 1
    assert lib.b200k_attn_supported(48, 4096) == 0 and lib.b200k_attn_supported(128, 200) == 1 and lib.b200k_attn_supported(128, 0) == 0
    assert lib.b200k_attn_bwd_supported(128, 4096) == 1 and lib.b200k_attn_bwd_supported(64, 256) == 1
    assert lib.b200k_attn_bwd_supported(32, 256) == 0 and lib.b200k_attn_bwd_supported(128, 192) == 1 and lib.b200k_attn_bwd_supported(64, 0) == 0
    assert lib.b200k_attn_bwd_bf16(16, 16, 16, 16, 16, 16, 16, 16, 16, 16, 1, 1, 256, 256, 0, 0.1, None) == _lib.ERR_UNSUPPORTED
    # argument checks of the backward come before any device work
    assert lib.b200k_attn_bwd_bf16(16, 16, 16, 16, 16, 16, 16, 16, 16, 16, 0, 1, 256, 128, 0, 0.1, None) == _lib.ERR_INVALID_ARG
    assert lib.b200k_attn_bwd_bf16(16, 16, 16, 16, 16, 16, 16, 16, None, 16, 1, 1, 256, 128, 0, 0.1, None) == _lib.ERR_INVALID_ARG
    assert "null" in _lib.last_error()
    assert lib.b200k_attn_bwd_bf16(16, 16, 16, 16, 16, 16, 16, 24, 16, 16, 1, 1, 256, 128, 0, 0.1, None) == _lib.ERR_INVALID_ARG
    assert "16-byte" in _lib.last_error()
    assert lib.b200k_attn_bwd_bf16(16, 16, 16, 16, 16, 16, 16, 16, 16, 16, 1, 1, 256, 128, 0, 0.0, None) == _lib.ERR_INVALID_ARG
    assert lib.b200k_attn_bwd_bf16(16, 16, 16, 16, 16, 16, 16, 16, 16, 16, 2 ** 20, 2 ** 11, 2 ** 10, 128, 0, 0.1, None) == _lib.ERR_INVALID_ARG
    assert "2^31" in _lib.last_error()
    assert lib.b200k_launch(b"no_such_kernel", 1, 1, 1, None, None, 0) == _lib.ERR_UNSUPPORTED
    assert lib.b200k_launch(b"add_kernel", 0, 1, 1, None, None, 0) == _lib.ERR_INVALID_ARG
    assert lib.b200k_launch(b"memcpy_kernel:XBLOCK=64", 1, 1, 1, None, None, 0) == _lib.ERR_INVALID_ARG   # no arguments
    assert lib.b200k_copy_f32(None, None, 4, 64, None) == _lib.ERR_INVALID_ARG and "null" in _lib.last_error()
    assert lib.b200k_copy_f32(None, None, 0, 64, None) == _lib.OK                                       # nothing to copy
    with pytest.raises(_lib.B200KError):
        _lib.check(lib.b200k_launch(b"add_kernel", 1, 1, 1, None, None, 0))  # wrong argument count
