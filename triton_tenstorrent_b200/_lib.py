"""ctypes binding of libb200kernels.so (the C-ABI declared in include/b200k.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, Union, c_char, c_char_p, c_float, c_int, c_int32, c_int64, c_uint32, c_void_p
from pathlib import Path

# B200K_LIBRARY selects another build of the same library (e.g. one compiled with debug defines).
LIB_PATH = Path(os.environ.get("B200K_LIBRARY") or Path(__file__).resolve().parent / "libb200kernels.so")

OK = 0
ERR_INVALID_ARG = -1
ERR_CUDA = -2
ERR_UNSUPPORTED = -3
ERR_NO_DEVICE = -4
ERR_DEVICE_TIMEOUT = -5

BIAS_NONE, BIAS_ROW_F32, BIAS_FULL_BF16 = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_LEAKY_RELU = 0, 1, 2
ARG_PTR, ARG_I32, ARG_I64, ARG_F32 = 0, 1, 2, 3


class B200KError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"b200k error {code}: {message}")
        self.code = code
        self.message = message


class _ArgValue(Union):
    _fields_ = [("ptr", c_void_p), ("i32", c_int32), ("i64", c_int64), ("f32", c_float)]


class Arg(Structure):
    """b200k_arg: one entry of the flattened launch argument list."""
    _fields_ = [("kind", c_int32), ("_pad", c_int32), ("v", _ArgValue)]


class IpcHandle(Structure):
    """b200k_ipc_handle: 88 bytes that describe an exported device allocation."""
    _fields_ = [("handle", ctypes.c_ubyte * 64), ("offset", c_int64), ("size", c_int64), ("device", c_int32),
                ("_pad", c_int32)]


class Props(Structure):
    """b200k_props."""
    _fields_ = [
        ("multiprocessor_count", c_int32),
        ("max_shared_mem", c_int32),
        ("max_num_regs", c_int32),
        ("warp_size", c_int32),
        ("cc_major", c_int32),
        ("cc_minor", c_int32),
        ("total_mem", c_int64),
        ("name", c_char * 128),
    ]


# name -> (restype, argtypes); mirrors include/b200k.h one to one.
SIGNATURES = {
    "b200k_version": (c_int, []),
    "b200k_last_error": (c_char_p, []),
    "b200k_add_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "b200k_add_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "b200k_sin_f32": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "b200k_copy_f32": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "b200k_mul_add_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "b200k_matmul_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                                  c_void_p, c_int, c_int64, c_int, c_int, c_void_p]),
    "b200k_matmul_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                                 c_void_p, c_int, c_int64, c_int, c_int, c_void_p]),
    "b200k_matmul_bf16_multi": (c_int, [c_void_p, c_void_p, POINTER(c_void_p), c_int, c_int, c_int, c_int, c_int64,
                                        c_int64, c_int64, c_void_p, c_int, c_int64, c_int, c_int, c_void_p]),
    "b200k_matmul_tile32": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "b200k_attn_fwd_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                    c_int, c_float, c_void_p]),
    "b200k_attn_fwd_bf16_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                            c_float, c_void_p]),
    "b200k_attn_noalloc_status": (c_int, [c_void_p, POINTER(c_uint32)]),
    "b200k_attn_noalloc_selftest": (c_int, [c_int64, c_void_p]),
    "b200k_attn_fwd_bf16_multi": (c_int, [c_void_p, c_void_p, c_void_p, POINTER(c_void_p), c_int, c_void_p, c_int, c_int,
                                          c_int, c_int, c_int, c_float, c_void_p]),
    "b200k_attn_causal_schedule": (c_int, [c_int, c_int, c_int, c_int, POINTER(c_int), c_int, POINTER(c_int)]),
    "b200k_attn_supported": (c_int, [c_int, c_int]),
    "b200k_attn_bwd_bf16": (c_int, [c_void_p] * 10 + [c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]),
    "b200k_attn_bwd_supported": (c_int, [c_int, c_int]),
    "b200k_launch": (c_int, [c_char_p, c_int, c_int, c_int, c_void_p, POINTER(Arg), c_int]),
    "b200k_device_props": (c_int, [c_int, POINTER(Props)]),
    "b200k_ipc_export": (c_int, [c_void_p, POINTER(IpcHandle)]),
    "b200k_ipc_open": (c_int, [POINTER(IpcHandle), POINTER(c_void_p)]),
    "b200k_block_range": (c_int, [c_int64, c_int, c_int, POINTER(c_int64), POINTER(c_int64)]),
    "b200k_matmul_tail_plan": (c_int, [c_int, c_int, c_int, c_int, POINTER(c_int)]),
    "b200k_device_status": (c_int, [c_void_p, POINTER(c_uint32)]),
    "b200k_selftest_wait_timeout": (c_int, [c_int64, c_void_p]),
    "b200k_launch_count": (c_int64, []),
}

_lib = None


def load() -> ctypes.CDLL:
    """Loads the shared library (once) and types every entry point.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m triton_tenstorrent_b200.build` "
            "(there is no CPU or PyTorch fallback for these kernels)")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    msg = load().b200k_last_error()
    return msg.decode() if msg else ""


def check(code: int) -> None:
    if code != OK:
        raise B200KError(code, last_error())
