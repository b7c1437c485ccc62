"""ctypes front end of the CPU oracle (oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke test of __graft_entry__ and the cpu-baseline / reference legs of bench.py may
import this module; the shipped package never does.  Tensors are CPU torch tensors; bf16 / fp16
tensors are passed as their 16-bit patterns.
"""
from __future__ import annotations

import ctypes
import subprocess
from ctypes import POINTER, c_float, c_int, c_int64, c_uint32, c_void_p
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
_lib = None


def build(force: bool = False) -> None:
    """Compiles oracle.c with the Makefile beside it."""
    if force:
        subprocess.run(["make", "-C", str(HERE), "clean"], check=True, capture_output=True)
    subprocess.run(["make", "-C", str(HERE)], check=True, capture_output=True)


def _has_avx2() -> bool:
    try:
        flags = Path("/proc/cpuinfo").read_text()
        return " avx2" in flags and " fma" in flags
    except OSError:
        return False


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    name = "liboracle_avx2.so" if _has_avx2() else "liboracle_base.so"
    path = HERE / name
    if not path.exists():
        build()
    lib = ctypes.CDLL(str(path))
    lib.oracle_max_threads.restype = c_int
    lib.oracle_set_threads.argtypes = [c_int]
    lib.oracle_set_threads.restype = None
    lib.oracle_block_range.argtypes = [c_int64, c_int, c_int, POINTER(c_int64), POINTER(c_int64)]
    lib.oracle_add_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int]
    lib.oracle_add_loop.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int]
    lib.oracle_sin_f32.argtypes = [c_void_p, c_void_p, c_int64, c_int, c_int]
    lib.oracle_memcpy_f32.argtypes = [c_void_p, c_void_p, c_int64, c_int, c_int]
    lib.oracle_sin_f64_to_f32.argtypes = [c_void_p, c_void_p, c_int64]
    lib.oracle_mul_add_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int]
    lib.oracle_golden_matmul.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int,
                                         c_void_p, c_void_p, c_int]
    lib.oracle_golden_matmul_naive.argtypes = [c_void_p, c_void_p, c_void_p, c_uint32, c_uint32, c_uint32]
    lib.oracle_matmul_kernel_tile32.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int]
    lib.oracle_attn_fwd_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                         c_int, c_float, c_int, c_int]
    lib.oracle_attn_bwd_bf16.argtypes = [c_void_p] * 9 + [c_int, c_int, c_int, c_int, c_int, c_float]
    lib.oracle_attn_bwd_bf16.restype = None
    for fn in ("oracle_block_range", "oracle_add_f32", "oracle_add_loop", "oracle_sin_f32", "oracle_memcpy_f32", "oracle_sin_f64_to_f32", "oracle_mul_add_f32",
               "oracle_golden_matmul", "oracle_golden_matmul_naive", "oracle_matmul_kernel_tile32", "oracle_attn_fwd_bf16"):
        getattr(lib, fn).restype = None
    _lib = lib
    return lib


def max_threads() -> int:
    return load().oracle_max_threads()


def use_all_cores() -> int:
    """Lets OpenMP use every host core even if OMP_NUM_THREADS says otherwise; returns the thread count."""
    import os
    load().oracle_set_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    return max_threads()


def _cpu(t: torch.Tensor, dtype=None) -> torch.Tensor:
    assert not t.is_cuda, "the oracle works on host tensors"
    if dtype is not None:
        assert t.dtype == dtype, f"expected {dtype}, got {t.dtype}"
    return t.contiguous()


def block_range(num_blocks: int, workers: int, w: int):
    s, e = c_int64(), c_int64()
    load().oracle_block_range(num_blocks, workers, w, ctypes.byref(s), ctypes.byref(e))
    return s.value, e.value


def add(x, y, block: int = 1024, workers: int = 0):
    x, y = _cpu(x, torch.float32), _cpu(y, torch.float32)
    out = torch.empty_like(x)
    load().oracle_add_f32(x.data_ptr(), y.data_ptr(), out.data_ptr(), x.numel(), block, workers)
    return out


def add_loop(x, y, row_count: int, grid: int, block: int = 1024, fill: float = 0.0):
    """The row_count-loop form of add_kernel (python/tutorials/01-vector-add.loop.py:29-66), fp32 or bf16.
    Elements that no program owns keep `fill`."""
    assert x.dtype == y.dtype and x.dtype in (torch.float32, torch.bfloat16)
    x, y = _cpu(x), _cpu(y)
    out = torch.full_like(x, fill)
    load().oracle_add_loop(x.data_ptr(), y.data_ptr(), out.data_ptr(), x.numel(), row_count, block, grid,
                           0 if x.dtype == torch.float32 else 1)
    return out


def sin(x, block: int = 1024, workers: int = 0):
    x = _cpu(x, torch.float32)
    out = torch.empty_like(x)
    load().oracle_sin_f32(x.data_ptr(), out.data_ptr(), x.numel(), block, workers)
    return out


def memcpy(x, xblock: int = 2048, workers: int = 0):
    """memcpy_kernel of python/tutorials/gluon/01-intro.py:84-93, block by block."""
    x = _cpu(x, torch.float32)
    out = torch.full_like(x, float("nan"))
    load().oracle_memcpy_f32(x.data_ptr(), out.data_ptr(), x.numel(), xblock, workers)
    return out


def sin_correctly_rounded(x):
    x = _cpu(x, torch.float32)
    out = torch.empty_like(x)
    load().oracle_sin_f64_to_f32(x.data_ptr(), out.data_ptr(), x.numel())
    return out


def mul_add(x, y, z, block: int = 1024, workers: int = 0):
    x, y, z = (_cpu(t, torch.float32) for t in (x, y, z))
    out = torch.empty_like(x)
    load().oracle_mul_add_f32(x.data_ptr(), y.data_ptr(), z.data_ptr(), out.data_ptr(), x.numel(), block, workers)
    return out


_ACT = {"": 0, None: 0, "none": 0, "relu": 1, "leaky_relu": 2}


def golden_matmul(a, b, bias=None, mode: int = 0, activation=""):
    """mode 0: C = h(act(acc)); 1: h(acc + bias[M,N]); 2: h(h(acc) + bias[M,N]); 3: h(act(acc + bias[N] fp32))."""
    assert a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16)
    dtype_flag = 0 if a.dtype == torch.bfloat16 else 1
    a, b = _cpu(a), _cpu(b)
    M, K = a.shape
    K2, N = b.shape
    assert K == K2
    out = torch.empty((M, N), dtype=a.dtype)
    bias_full = bias_row = None
    if mode in (1, 2):
        bias_full = _cpu(bias, a.dtype)
        assert bias_full.shape == (M, N)
    elif mode == 3:
        bias_row = _cpu(bias, torch.float32)
        assert bias_row.shape == (N,)
    load().oracle_golden_matmul(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, dtype_flag, mode,
                                bias_full.data_ptr() if bias_full is not None else None,
                                bias_row.data_ptr() if bias_row is not None else None, _ACT[activation])
    return out


def tilize(t, tile: int = 32):
    """Row-major [R,S] -> the same shape whose MEMORY holds contiguous tile x tile tiles in row-major tile order
    (the layout examples/matmul/03-matrix-multiplication.py:333-386 addresses)."""
    R, S = t.shape
    assert R % tile == 0 and S % tile == 0
    return t.reshape(R // tile, tile, S // tile, tile).permute(0, 2, 1, 3).contiguous().view(R, S)


def untilize(t, tile: int = 32):
    """Inverse of tilize."""
    R, S = t.shape
    assert R % tile == 0 and S % tile == 0
    return t.reshape(R // tile, S // tile, tile, tile).permute(0, 2, 1, 3).contiguous().view(R, S)


def matmul_kernel_tile32(a_tiled, b_tiled, activation=""):
    """The reference's pointer-based matmul_kernel on tile-major buffers (tile-major result)."""
    assert a_tiled.dtype == b_tiled.dtype and a_tiled.dtype in (torch.bfloat16, torch.float16)
    a, b = _cpu(a_tiled), _cpu(b_tiled)
    M, K = a.shape
    K2, N = b.shape
    assert K == K2 and M % 32 == 0 and N % 32 == 0 and K % 32 == 0
    out = torch.empty((M, N), dtype=a.dtype)
    load().oracle_matmul_kernel_tile32(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K,
                                       0 if a.dtype == torch.bfloat16 else 1, _ACT[activation])
    return out


def golden_matmul_naive(a, b):
    """The reference's golden_matmul loop exactly as written (bf16); slow, used as the timed CPU baseline."""
    a, b = _cpu(a, torch.bfloat16), _cpu(b, torch.bfloat16)
    M, K = a.shape
    _, N = b.shape
    out = torch.empty((M, N), dtype=torch.bfloat16)
    load().oracle_golden_matmul_naive(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K)
    return out


def attention(q, k, v, causal: bool, sm_scale: float, BLOCK_M: int = 128, BLOCK_N: int = 128):
    """Returns (O bf16 [Z,H,S,D], M fp32 [Z,H,S]) computed block by block like the reference kernel."""
    q, k, v = (_cpu(t, torch.bfloat16) for t in (q, k, v))
    Z, H, S, D = q.shape
    o = torch.empty_like(q)
    M = torch.empty((Z, H, S), dtype=torch.float32)
    load().oracle_attn_fwd_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), M.data_ptr(), Z, H, S, D,
                                1 if causal else 0, float(sm_scale), BLOCK_M, BLOCK_N)
    return o, M


def attention_backward(q, k, v, o, d_o, M, causal: bool, sm_scale: float):
    """(dq, dk, dv) bf16 from q, k, v, the forward's o and M, and the gradient of o.  PARITY UNPINNED: the reference has
    no backward kernel; this restates the Triton tutorial's algorithm in the forward's conventions (see oracle.c)."""
    q, k, v, o, d_o = (_cpu(t, torch.bfloat16) for t in (q, k, v, o, d_o))
    M = _cpu(M, torch.float32)
    Z, H, S, D = q.shape
    assert D <= 256
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    load().oracle_attn_bwd_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), M.data_ptr(),
                                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), Z, H, S, D, 1 if causal else 0, float(sm_scale))
    return dq, dk, dv


# ---- error metrics used by the parity tests -----------------------------------------------------
def ulp_diff_f32(a: torch.Tensor, b: torch.Tensor) -> int:
    """Largest distance in units in the last place between two fp32 tensors (finite values)."""
    ia = a.contiguous().view(torch.int32).to(torch.int64)
    ib = b.contiguous().view(torch.int32).to(torch.int64)
    # map the sign-magnitude float ordering onto a monotonic integer line
    ia = torch.where(ia < 0, -(ia & 0x7FFFFFFF), ia)
    ib = torch.where(ib < 0, -(ib & 0x7FFFFFFF), ib)
    return int((ia - ib).abs().max().item()) if a.numel() else 0


def rel_frobenius(x: torch.Tensor, ref: torch.Tensor) -> float:
    x, ref = x.double(), ref.double()
    return float((x - ref).norm() / ref.norm())


def pcc(x: torch.Tensor, ref: torch.Tensor) -> float:
    """Pearson correlation, the reference's own acceptance gate (examples/01-sin-kernel.py:40-49)."""
    x, ref = x.double().reshape(-1), ref.double().reshape(-1)
    if x.numel() < 2 or x.std() == 0 or ref.std() == 0:
        return 1.0 if torch.allclose(x, ref) else 0.0
    return float(torch.corrcoef(torch.stack([x, ref]))[0, 1])
