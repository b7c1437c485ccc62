"""Host wrappers with the names and argument meaning of the reference examples' wrappers.

Each function validates like the reference wrapper it mirrors, allocates the output with torch and
calls the C-ABI (include/b200k.h) on the current CUDA stream.  Tensors may live on the GPU (the
normal case) or on the host: host tensors are copied to the current device, computed there and the
result is copied back, which is what the reference's D2M launcher does on every launch
(backend/driver.py:350-381).  There is no CPU compute path.
"""
from __future__ import annotations

import contextlib
import ctypes

import torch

from . import _lib

__all__ = ["add", "add_loop", "sin", "memcpy", "mul_add", "matmul", "tilize", "untilize", "matmul_tma", "matmul_tma_host_rows", "matmul_multi", "matmul_fused", "matmul_tma_fused", "attention", "attention_multi",
           "attention_with_lse", "attention_backward", "device_status"]


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """Handle of the current CUDA stream of the current device (the raw query avoids building a Stream object on
    every launch, which matters for the launch-bound sizes)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


_NO_SWITCH = contextlib.nullcontext()


def _on(device):
    """Context that makes `device` current for a C-ABI call; free when it already is (the usual case)."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(device)


def _require_cuda():
    if not torch.cuda.is_available():
        raise RuntimeError("triton_tenstorrent_b200 needs a CUDA device (sm_100a); there is no CPU fallback")


def _to_device(t: torch.Tensor) -> torch.Tensor:
    if t.is_cuda:
        return t
    _require_cuda()
    return t.to("cuda", non_blocking=True)


def _like_input(result: torch.Tensor, ref: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """Returns `result` on the device `ref` lives on (host inputs get a host result).  With `out`
    (an extension over the reference wrappers) the result is copied into that tensor instead, e.g. a
    pinned host buffer the caller reuses between calls; the copy is complete on return."""
    if out is not None:
        if out.shape != result.shape or out.dtype != result.dtype:
            raise ValueError(f"out must be {tuple(result.shape)} {result.dtype}")
        if out.data_ptr() != result.data_ptr():
            out.copy_(result, non_blocking=True)
            if not out.is_cuda:
                torch.cuda.current_stream().synchronize()
        return out
    if ref.is_cuda:
        return result
    return result.to("cpu")


def _elementwise_check(name, *tensors, dtypes=(torch.float32,)):
    t0 = tensors[0]
    for t in tensors:
        if t.dtype not in dtypes:
            raise TypeError(f"{name}: {' or '.join(str(d) for d in dtypes)} tensors expected, got {t.dtype}")
        if t.dtype != t0.dtype:
            raise TypeError(f"{name}: mixed dtypes {t0.dtype} and {t.dtype}")
        if t.shape != t0.shape:
            raise ValueError(f"{name}: shape mismatch {tuple(t.shape)} vs {tuple(t0.shape)}")
        if t.device != t0.device:
            raise ValueError(f"{name}: tensors on different devices")


def add(x: torch.Tensor, y: torch.Tensor, BLOCK_SIZE: int = 1024) -> torch.Tensor:
    """out = x + y, fp32 or bf16.  Mirrors add(), python/tutorials/01-vector-add.py:62-78 (fp32) and
    python/tutorials/01-vector-add.loop.py:74-97 (which runs bf16 tensors)."""
    _elementwise_check("add", x, y, dtypes=(torch.float32, torch.bfloat16))
    lib = _lib.load()
    xd, yd = _to_device(x).contiguous(), _to_device(y).contiguous()
    out = torch.empty_like(xd)
    entry = lib.b200k_add_f32 if xd.dtype == torch.float32 else lib.b200k_add_bf16
    with _on(xd.device):
        _lib.check(entry(xd.data_ptr(), yd.data_ptr(), out.data_ptr(), out.numel(), BLOCK_SIZE, _stream()))
    return _like_input(out, x)


def add_loop(x: torch.Tensor, y: torch.Tensor, n_cores: int = 130, BLOCK_SIZE: int = 1024) -> torch.Tensor:
    """out = x + y launched like add() of python/tutorials/01-vector-add.loop.py:74-97: at most `n_cores`
    programs, each walking row_count = cdiv(cdiv(n, BLOCK_SIZE), n_cores) consecutive blocks."""
    from . import kernels
    _elementwise_check("add_loop", x, y, dtypes=(torch.float32, torch.bfloat16))
    xd, yd = _to_device(x).contiguous(), _to_device(y).contiguous()
    out = torch.empty_like(xd)
    n_elements = out.numel()
    if n_elements == 0:
        return _like_input(out, x)
    n_rows = -(-n_elements // BLOCK_SIZE)
    row_count = -(-n_rows // n_cores)
    if n_rows < n_cores:
        n_cores = n_rows
    with _on(xd.device):
        kernels.add_kernel_loop[lambda meta: (n_cores,)](xd, yd, out, n_elements, row_count, BLOCK_SIZE=BLOCK_SIZE,
                                                         num_warps=1)
    return _like_input(out, x)


def sin(x: torch.Tensor, BLOCK_SIZE: int = 1024) -> torch.Tensor:
    """out = sin(x) (fp32).  Mirrors sin(), examples/01-sin-kernel.py:32-37."""
    _elementwise_check("sin", x)
    lib = _lib.load()
    xd = _to_device(x).contiguous()
    out = torch.empty_like(xd)
    with _on(xd.device):
        _lib.check(lib.b200k_sin_f32(xd.data_ptr(), out.data_ptr(), out.numel(), BLOCK_SIZE, _stream()))
    return _like_input(out, x)


def memcpy(input: torch.Tensor, output: torch.Tensor = None, XBLOCK: int = 2048) -> torch.Tensor:
    """output[i] = input[i] (fp32, bit for bit).  Mirrors memcpy(input, output, XBLOCK), python/tutorials/gluon/01-intro.py:96-99;
    without `output` a new tensor is returned."""
    _elementwise_check("memcpy", input)
    lib = _lib.load()
    xd = _to_device(input).contiguous()
    if output is None:
        out = torch.empty_like(xd)
    else:
        if output.dtype != torch.float32 or output.numel() != input.numel() or not output.is_contiguous():
            raise ValueError("memcpy: output must be a contiguous fp32 tensor with as many elements as input")
        out = _to_device(output)
    with _on(xd.device):
        _lib.check(lib.b200k_copy_f32(xd.data_ptr(), out.data_ptr(), xd.numel(), XBLOCK, _stream()))
    if output is not None and not output.is_cuda:
        output.copy_(out)
        return output
    return out if output is not None else _like_input(out, input)


def mul_add(x: torch.Tensor, y: torch.Tensor, z: torch.Tensor, BLOCK_SIZE: int = 1024) -> torch.Tensor:
    """out = x * y + z (fp32, two roundings).  Mirrors python/tutorials/01-vector-mul-add.py."""
    _elementwise_check("mul_add", x, y, z)
    lib = _lib.load()
    xd, yd, zd = (_to_device(t).contiguous() for t in (x, y, z))
    out = torch.empty_like(xd)
    with _on(xd.device):
        _lib.check(lib.b200k_mul_add_f32(xd.data_ptr(), yd.data_ptr(), zd.data_ptr(), out.data_ptr(), out.numel(),
                                         BLOCK_SIZE, _stream()))
    return _like_input(out, x)


_ACTIVATIONS = {"": _lib.ACT_NONE, None: _lib.ACT_NONE, "none": _lib.ACT_NONE, "relu": _lib.ACT_RELU,
                "leaky_relu": _lib.ACT_LEAKY_RELU}


def _row_major_2d(t: torch.Tensor, name: str) -> torch.Tensor:
    """A 2-D bf16 / fp16 view the TMA path accepts: unit inner stride, 16-byte aligned rows and base."""
    if t.dim() != 2:
        raise ValueError(f"{name}: 2-D tensor expected, got {t.dim()}-D")
    if t.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"{name}: bf16 or fp16 expected, got {t.dtype}")
    if t.stride(1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0 or t.stride(0) < t.shape[1]:
        if t.shape[1] % 8 != 0:
            raise ValueError(f"{name}: the row length must be a multiple of 8 elements (16-byte rows, the same "
                             f"constraint a tensor descriptor has); got shape {tuple(t.shape)}")
        t = t.contiguous()
    return t


_HOST_CHUNK_ROWS = 1024     # rows of A / C per piece of the host-tensor pipeline (a multiple of the 256-row tile)
_copy_streams = {}


def _side_streams(device):
    """Two extra streams per device: host-to-device and device-to-host copies of the host-tensor pipeline."""
    key = torch.device(device).index
    if key not in _copy_streams:
        _copy_streams[key] = (torch.cuda.Stream(device=device), torch.cuda.Stream(device=device))
    return _copy_streams[key]


def matmul_tma_host_rows(a: torch.Tensor, b_dev: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """C = A.B for a HOST A (and host result) against a B that is already resident on the current device:
    the row-block pipeline of matmul_tma's host path without the upload of B.  Used when B reaches the
    GPU some other way, e.g. gathered over NVLink from the other GPUs of the box."""
    if a.is_cuda or not b_dev.is_cuda:
        raise ValueError("matmul_tma_host_rows: a must be a host tensor and b_dev a CUDA tensor")
    if a.shape[0] < 2 * _HOST_CHUNK_ROWS:
        c = _matmul_call(a, b_dev)
        return _like_input(c, a, out)
    return _matmul_host_streamed(a, None, out, None, _lib.BIAS_NONE, _lib.ACT_NONE, 0, b_dev=b_dev)


def _matmul_host_streamed(a, b, out, bias, bias_kind, act, round_before_bias, b_dev=None):
    """C = epilogue(A.B) for HOST operands, as a three-stage pipeline over row blocks of A and C:
    while block i is multiplied, block i+1 of A travels to the device and block i-1 of C travels back
    (PCIe is full duplex), so a call costs about the upload of B plus the upload of A instead of the
    sum of all copies and the kernel.  Pinned host tensors make the copies asynchronous; pageable ones
    still work (torch stages them).  Returns a host tensor (`out` if given)."""
    _require_cuda()
    device = torch.device("cuda", torch.cuda.current_device())
    M, K = a.shape
    N = b.shape[1] if b_dev is None else b_dev.shape[1]
    main = torch.cuda.current_stream(device)
    s_in, s_out = _side_streams(device)
    if out is None:
        out = torch.empty((M, N), dtype=a.dtype, pin_memory=True)
    elif tuple(out.shape) != (M, N) or out.dtype != a.dtype or out.is_cuda:
        raise ValueError(f"out must be a host {a.dtype} [{M},{N}] tensor")
    a_dev = torch.empty((M, K), dtype=a.dtype, device=device)
    c_dev = torch.empty((M, N), dtype=a.dtype, device=device)
    s_in.wait_stream(main)
    s_out.wait_stream(main)
    with torch.cuda.stream(s_in):
        if b_dev is None:      # otherwise B is already on the device (ordered on the main stream)
            b_dev = b.to(device, non_blocking=True)
        bias_dev = bias.to(device, non_blocking=True) if bias is not None else None
    blocks = [(r, min(r + _HOST_CHUNK_ROWS, M)) for r in range(0, M, _HOST_CHUNK_ROWS)]
    for (r0, r1) in blocks:
        with torch.cuda.stream(s_in):
            a_dev[r0:r1].copy_(a[r0:r1], non_blocking=True)
            ready = s_in.record_event()
        main.wait_event(ready)
        _matmul_call(a_dev[r0:r1], b_dev, c=c_dev[r0:r1],
                     bias=(bias_dev[r0:r1] if bias_kind == _lib.BIAS_FULL_BF16 else bias_dev),
                     bias_kind=bias_kind, act=act, round_before_bias=round_before_bias)
        done = main.record_event()
        s_out.wait_event(done)
        with torch.cuda.stream(s_out):
            out[r0:r1].copy_(c_dev[r0:r1], non_blocking=True)
    main.wait_stream(s_out)
    s_out.synchronize()
    for t in (a_dev, c_dev, b_dev):      # the side streams used these allocations
        t.record_stream(s_in)
        t.record_stream(s_out)
    return out


def _matmul_call(a, b, c=None, bias=None, bias_kind=_lib.BIAS_NONE, act=_lib.ACT_NONE, round_before_bias=0):
    assert a.shape[1] == b.shape[0], "Incompatible dimensions"
    assert a.dtype == b.dtype, "Incompatible dtypes"
    lib = _lib.load()
    ad, bd = _row_major_2d(_to_device(a), "a"), _row_major_2d(_to_device(b), "b")
    M, K = ad.shape
    _, N = bd.shape
    if N % 8 != 0:
        raise ValueError(f"matmul: N must be a multiple of 8 (16-byte rows of C); got {N}")
    dtype = ad.dtype
    if c is None:
        c = torch.empty((M, N), device=ad.device, dtype=dtype)
    elif (tuple(c.shape) != (M, N) or c.dtype != dtype or not c.is_cuda or c.device != ad.device
          or c.stride(1) != 1 or c.stride(0) % 8 != 0 or c.data_ptr() % 16 != 0):
        raise ValueError(f"matmul: the output must be a {dtype} [{M},{N}] tensor on {ad.device} with unit inner "
                         "stride and 16-byte aligned rows")
    bias_ptr, ldbias = 0, 0
    if bias_kind == _lib.BIAS_ROW_F32:
        bias = _to_device(bias).contiguous()
        if bias.dtype != torch.float32 or bias.shape != (N,):
            raise ValueError(f"bias must be fp32 [N={N}], got {bias.dtype} {tuple(bias.shape)}")
        bias_ptr = bias.data_ptr()
    elif bias_kind == _lib.BIAS_FULL_BF16:
        bias = _to_device(bias)
        assert bias.shape == (M, N), "Incompatible bias dimensions"
        if bias.dtype != dtype:
            raise TypeError(f"bias must be {dtype} [M,N] like the operands, got {bias.dtype}")
        if bias.stride(1) != 1:
            bias = bias.contiguous()
        bias_ptr, ldbias = bias.data_ptr(), bias.stride(0)
    entry = lib.b200k_matmul_f16 if dtype == torch.float16 else lib.b200k_matmul_bf16
    with _on(ad.device):
        _lib.check(entry(ad.data_ptr(), bd.data_ptr(), c.data_ptr(), M, N, K, ad.stride(0), bd.stride(0),
                         c.stride(0), bias_ptr, bias_kind, ldbias, act, round_before_bias, _stream()))
    return c


def matmul_multi(a: torch.Tensor, b: torch.Tensor, dests, bias: torch.Tensor = None, activation: str = "",
                 remote_ptrs=()):
    """C = act(A.B [+ bias[N]]) stored by the kernel's epilogue into every tensor of `dests` (bf16 [M,N] tensors with
    one common row stride) and to every address of `remote_ptrs` (device addresses of [M,N] blocks with that same row
    stride, e.g. row blocks of other GPUs' buffers mapped by sharding.GatheredRows); at most 8 destinations in
    all.  With remote destinations the matmul doubles as the sending side of an all-gather of C.  Readers of
    remote destinations must be ordered after the launch by the caller.  Returns dests[0]."""
    if activation not in _ACTIVATIONS:
        raise ValueError(f"unknown activation {activation!r}")
    dests, remote_ptrs = list(dests), [int(p) for p in remote_ptrs]
    if len(dests) < 1 or len(dests) + len(remote_ptrs) > 8:
        raise ValueError(f"matmul_multi: 1..8 destinations expected, got {len(dests)} + {len(remote_ptrs)}")
    assert a.shape[1] == b.shape[0], "Incompatible dimensions"
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("matmul_multi: bf16 operands expected")
    if not (a.is_cuda and b.is_cuda):
        raise ValueError("matmul_multi: operands must live on the GPU")
    lib = _lib.load()
    ad, bd = _row_major_2d(a, "a"), _row_major_2d(b, "b")
    M, K = ad.shape
    _, N = bd.shape
    ldc = dests[0].stride(0)
    for i, d in enumerate(dests):
        if (not d.is_cuda or d.device != ad.device or d.dtype != torch.bfloat16 or tuple(d.shape) != (M, N)
                or d.stride(1) != 1 or d.stride(0) != ldc or ldc % 8 != 0 or d.data_ptr() % 16 != 0):
            raise ValueError(f"matmul_multi: destination {i} must be a bf16 [{M},{N}] tensor on {ad.device} with unit "
                             f"inner stride, row stride {ldc} (a multiple of 8) and a 16-byte aligned base")
    for p in remote_ptrs:
        if p == 0 or p % 16 != 0:
            raise ValueError("matmul_multi: remote destinations must be non-null and 16-byte aligned")
    bias_ptr, bias_kind = 0, _lib.BIAS_NONE
    if bias is not None:
        bias = bias.contiguous()
        if bias.dtype != torch.float32 or tuple(bias.shape) != (N,) or bias.device != ad.device:
            raise ValueError(f"bias must be fp32 [N={N}] on {ad.device}")
        bias_ptr, bias_kind = bias.data_ptr(), _lib.BIAS_ROW_F32
    all_ptrs = [d.data_ptr() for d in dests] + remote_ptrs
    ptrs = (ctypes.c_void_p * len(all_ptrs))(*all_ptrs)
    with _on(ad.device):
        _lib.check(lib.b200k_matmul_bf16_multi(ad.data_ptr(), bd.data_ptr(), ptrs, len(all_ptrs), M, N, K, ad.stride(0),
                                               bd.stride(0), ldc, bias_ptr, bias_kind, 0, _ACTIVATIONS[activation], 0,
                                               _stream()))
    return dests[0]


def matmul_tma(a: torch.Tensor, b: torch.Tensor, warp_specialize: bool = True, out: torch.Tensor = None) -> torch.Tensor:
    """C = A.B, bf16 (or fp16) in/out, fp32 accumulate.  Mirrors matmul_tma(a, b, warp_specialize),
    examples/matmul_tensor_descriptor/09-persistent-matmul.ttnn.py:146-173 (fp16 twin: 09-persistent-matmul.py:148-175).  `warp_specialize` is accepted for
    surface compatibility; the kernel is always warp-specialised."""
    if _host_pipeline_applies(a, b, out):
        return _matmul_host_streamed(a, b, out, None, _lib.BIAS_NONE, _lib.ACT_NONE, 0)
    return _like_input(_matmul_call(a, b, c=out if (out is not None and out.is_cuda) else None), a, out)


def _host_pipeline_applies(a, b, out, bias=None) -> bool:
    """Host operands, a host (or no) output, and enough rows for at least two pieces."""
    return (not a.is_cuda and not b.is_cuda and (out is None or not out.is_cuda) and (bias is None or not bias.is_cuda)
            and a.dim() == 2 and b.dim() == 2 and a.is_contiguous() and b.is_contiguous()
            and a.shape[0] >= 2 * _HOST_CHUNK_ROWS and a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0
            and a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16))


def tilize(t: torch.Tensor, tile: int = 32) -> torch.Tensor:
    """Row-major [R,S] -> a tensor of the same shape whose MEMORY holds contiguous tile x tile tiles, tiles in
    row-major order: the layout the reference's matmul_kernel addresses
    (examples/matmul/03-matrix-multiplication.py:333-344).  A layout helper in torch, not a kernel of this library."""
    R, S = t.shape
    if R % tile or S % tile:
        raise ValueError(f"tilize: shape {tuple(t.shape)} is not a whole number of {tile}x{tile} tiles")
    return t.reshape(R // tile, tile, S // tile, tile).permute(0, 2, 1, 3).contiguous().view(R, S)


def untilize(t: torch.Tensor, tile: int = 32) -> torch.Tensor:
    """Inverse of tilize: tile-major memory -> row-major."""
    R, S = t.shape
    if R % tile or S % tile:
        raise ValueError(f"untilize: shape {tuple(t.shape)} is not a whole number of {tile}x{tile} tiles")
    return t.reshape(R // tile, S // tile, tile, tile).permute(0, 2, 1, 3).contiguous().view(R, S)


def _matmul_tile32_call(a, b, act, c=None):
    """A, B, C are [M,K], [K,N], [M,N] tensors whose memory is tile-major (32 x 32 tiles)."""
    assert a.shape[1] == b.shape[0], "Incompatible dimensions"
    assert a.dtype == b.dtype, "Incompatible dtypes"
    lib = _lib.load()
    ad, bd = _to_device(a), _to_device(b)
    for name, t in (("a", ad), ("b", bd)):
        if t.dim() != 2 or t.dtype not in (torch.bfloat16, torch.float16):
            raise TypeError(f"{name}: 2-D bf16 or fp16 tensor expected")
        if not t.is_contiguous() or t.data_ptr() % 16 != 0:
            raise ValueError(f"{name}: a tile-major buffer must be contiguous and 16-byte aligned")
    M, K = ad.shape
    _, N = bd.shape
    if M % 32 or N % 32 or K % 32:
        raise ValueError(f"matmul: tile-major operands need M, N, K multiples of 32; got {M}, {N}, {K}")
    if c is None:
        c = torch.empty((M, N), device=ad.device, dtype=ad.dtype)
    elif (tuple(c.shape) != (M, N) or c.dtype != ad.dtype or not c.is_cuda or c.device != ad.device
          or not c.is_contiguous() or c.data_ptr() % 16 != 0):
        raise ValueError(f"matmul: the tile-major output must be a contiguous {ad.dtype} [{M},{N}] tensor on {ad.device}")
    with _on(ad.device):
        _lib.check(lib.b200k_matmul_tile32(ad.data_ptr(), bd.data_ptr(), c.data_ptr(), M, N, K, act,
                                           1 if ad.dtype == torch.float16 else 0, _stream()))
    return c


def matmul(a: torch.Tensor, b: torch.Tensor, activation: str = "", layout: str = "row") -> torch.Tensor:
    """C = act(A.B) with act in {"", "leaky_relu", "relu"} applied to the fp32 accumulator.
    Mirrors matmul(a, b, activation), examples/matmul/03-matrix-multiplication.py:403-421.
    layout="row": a, b and the result are ordinary row-major tensors.
    layout="tile32": the memory of a, b and of the result is tile-major (contiguous 32 x 32 tiles), which is how the
    reference kernel addresses its buffers (:333-386); see tilize / untilize."""
    assert a.is_contiguous(), "Matrix A must be contiguous"
    if activation not in _ACTIVATIONS:
        raise ValueError(f"unknown activation {activation!r}")
    if layout == "tile32":
        return _like_input(_matmul_tile32_call(a, b, _ACTIVATIONS[activation]), a)
    if layout != "row":
        raise ValueError(f"unknown layout {layout!r} (expected 'row' or 'tile32')")
    return _like_input(_matmul_call(a, b, act=_ACTIVATIONS[activation]), a)


def matmul_fused(a: torch.Tensor, b: torch.Tensor, bias: torch.Tensor, activation: str = "relu",
                 out: torch.Tensor = None) -> torch.Tensor:
    """C = act(A.B + bias[N]) in one kernel: fp32 bias add and activation on the accumulator, one downcast.
    This is the [N]-bias + ReLU epilogue of the fused-matmul workload."""
    if activation not in _ACTIVATIONS:
        raise ValueError(f"unknown activation {activation!r}")
    if _host_pipeline_applies(a, b, out, bias) and bias.dtype == torch.float32 and tuple(bias.shape) == (b.shape[1],):
        return _matmul_host_streamed(a, b, out, bias, _lib.BIAS_ROW_F32, _ACTIVATIONS[activation], 0)
    return _like_input(_matmul_call(a, b, c=out if (out is not None and out.is_cuda) else None, bias=bias,
                                    bias_kind=_lib.BIAS_ROW_F32, act=_ACTIVATIONS[activation]), a, out)


def matmul_tma_fused(a: torch.Tensor, b: torch.Tensor, bias: torch.Tensor, warp_specialize: bool = True,
                     round_before_bias: bool = True) -> torch.Tensor:
    """C = (A.B downcast) + bias[M,N].  Mirrors matmul_tma(a, b, bias, warp_specialize),
    python/tutorials/09-matmul-fused.py:151-181: the bias tile is added after the downcast (:139-146).
    round_before_bias=False gives the single rounding of the C++ golden (matmul_fused_add.cpp:49)."""
    return _like_input(_matmul_call(a, b, bias=bias, bias_kind=_lib.BIAS_FULL_BF16,
                                    round_before_bias=1 if round_before_bias else 0), a)


def attention_with_lse(q, k, v, causal, sm_scale, warp_specialize: bool = True):
    """Returns (O, M): the attention output and the fp32 base-2 log-sum-exp rows the reference saves for
    its backward (examples/fused-attn/06-fused-attention.py:238,269)."""
    HEAD_DIM_Q, HEAD_DIM_K, HEAD_DIM_V = q.shape[-1], k.shape[-1], v.shape[-1]
    assert HEAD_DIM_Q == HEAD_DIM_K and HEAD_DIM_K == HEAD_DIM_V
    assert HEAD_DIM_K in {16, 32, 64, 128, 256}
    if q.dim() != 4 or q.shape != k.shape or q.shape != v.shape:
        raise ValueError("attention: q, k, v must be [Z, H, N_CTX, HEAD_DIM] with equal shapes")
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise TypeError("attention: bf16 tensors expected")
    lib = _lib.load()
    Z, H, N_CTX, D = q.shape
    if not lib.b200k_attn_supported(D, N_CTX):
        raise NotImplementedError(f"attention: no sm_100a kernel for HEAD_DIM={D}, N_CTX={N_CTX}")
    qd, kd, vd = (_to_device(t).contiguous() for t in (q, k, v))
    o = torch.empty_like(qd)
    M = torch.empty((Z, H, N_CTX), device=qd.device, dtype=torch.float32)
    with _on(qd.device):
        _lib.check(lib.b200k_attn_fwd_bf16(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), M.data_ptr(),
                                           Z, H, N_CTX, D, 1 if causal else 0, float(sm_scale), _stream()))
    return _like_input(o, q), _like_input(M, q)


def attention_multi(q, k, v, causal, sm_scale, out: torch.Tensor, remote_ptrs=()):
    """O = attention(q, k, v) written by the kernel's epilogue into `out` (a contiguous bf16 [Z,H,N_CTX,D] tensor on
    q's device, e.g. this rank's block of a larger buffer) and to every device address of `remote_ptrs` (the same
    block inside other GPUs' buffers, mapped by sharding.GatheredRows); at most 8 destinations in all.  Returns
    (out, M)."""
    if q.dim() != 4 or q.shape != k.shape or q.shape != v.shape:
        raise ValueError("attention: q, k, v must be [Z, H, N_CTX, HEAD_DIM] with equal shapes")
    if any(t.dtype != torch.bfloat16 or not t.is_cuda for t in (q, k, v, out)):
        raise TypeError("attention_multi: bf16 CUDA tensors expected")
    remote_ptrs = [int(p) for p in remote_ptrs]
    if 1 + len(remote_ptrs) > 8:
        raise ValueError("attention_multi: at most 8 destinations")
    lib = _lib.load()
    Z, H, N_CTX, D = q.shape
    if not lib.b200k_attn_supported(D, N_CTX):
        raise NotImplementedError(f"attention: no sm_100a kernel for HEAD_DIM={D}, N_CTX={N_CTX}")
    if out.numel() != q.numel() or not out.is_contiguous() or out.device != q.device or out.data_ptr() % 16 != 0:
        raise ValueError("attention_multi: out must be a contiguous block of Z*H*N_CTX*D bf16 elements on q's device")
    for p in remote_ptrs:
        if p == 0 or p % 16 != 0:
            raise ValueError("attention_multi: remote destinations must be non-null and 16-byte aligned")
    qd, kd, vd = (t.contiguous() for t in (q, k, v))
    M = torch.empty((Z, H, N_CTX), device=qd.device, dtype=torch.float32)
    all_ptrs = [out.data_ptr()] + remote_ptrs
    ptrs = (ctypes.c_void_p * len(all_ptrs))(*all_ptrs)
    with _on(qd.device):
        _lib.check(lib.b200k_attn_fwd_bf16_multi(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), ptrs, len(all_ptrs),
                                                 M.data_ptr(), Z, H, N_CTX, D, 1 if causal else 0, float(sm_scale),
                                                 _stream()))
    return out, M


def attention_backward(q, k, v, o, M, d_o, causal, sm_scale):
    """(dq, dk, dv) from what the forward saved (q, k, v, o, M: examples/fused-attn/06-fused-attention.py:269) and the
    gradient of o.  The reference has no backward kernel; this is the consumer of its saved tensors (HEAD_DIM 64 or 128,
    N_CTX a multiple of 128)."""
    if q.dim() != 4 or any(t.shape != q.shape for t in (k, v, o, d_o)):
        raise ValueError("attention_backward: q, k, v, o, d_o must be [Z, H, N_CTX, HEAD_DIM] with equal shapes")
    if any(t.dtype != torch.bfloat16 for t in (q, k, v, o, d_o)) or M.dtype != torch.float32:
        raise TypeError("attention_backward: bf16 q, k, v, o, d_o and fp32 M expected")
    lib = _lib.load()
    Z, H, N_CTX, D = q.shape
    if tuple(M.shape) != (Z, H, N_CTX):
        raise ValueError("attention_backward: M must be [Z, H, N_CTX]")
    if not lib.b200k_attn_bwd_supported(D, N_CTX):
        raise NotImplementedError(f"attention backward: no sm_100a kernel for HEAD_DIM={D}, N_CTX={N_CTX} "
                                  "(HEAD_DIM 64 or 128)")
    qd, kd, vd, od, dod, Md = (_to_device(t).contiguous() for t in (q, k, v, o, d_o, M))
    dq, dk, dv = torch.empty_like(qd), torch.empty_like(qd), torch.empty_like(qd)
    delta = torch.empty((Z, H, N_CTX), device=qd.device, dtype=torch.float32)
    with _on(qd.device):
        _lib.check(lib.b200k_attn_bwd_bf16(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), od.data_ptr(), dod.data_ptr(),
                                           Md.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr(),
                                           Z, H, N_CTX, D, 1 if causal else 0, float(sm_scale), _stream()))
    return _like_input(dq, q), _like_input(dk, q), _like_input(dv, q)


class _attention(torch.autograd.Function):
    """The reference's `_attention` autograd function (examples/fused-attn/06-fused-attention.py:222-273) with the
    backward it lacks: forward saves (q, k, v, o, M) exactly as the reference does (:269)."""

    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale, warp_specialize=True):
        o, M = attention_with_lse(q, k, v, causal, sm_scale, warp_specialize)
        ctx.save_for_backward(q, k, v, o, M)
        ctx.sm_scale = sm_scale
        ctx.causal = causal
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, M = ctx.saved_tensors
        dq, dk, dv = attention_backward(q, k, v, o, M, d_o.contiguous(), ctx.causal, ctx.sm_scale)
        return dq, dk, dv, None, None, None


def attention(q, k, v, causal, sm_scale, warp_specialize: bool = True) -> torch.Tensor:
    """O = softmax(Q K^T sm_scale [+ causal mask]) V.  Mirrors _attention.forward / _attention.apply,
    examples/fused-attn/06-fused-attention.py:224-273; differentiable where the backward kernels apply."""
    if torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v)):
        return _attention.apply(q, k, v, causal, sm_scale, warp_specialize)
    return attention_with_lse(q, k, v, causal, sm_scale, warp_specialize)[0]


def device_status() -> int:
    """Synchronises the current stream and returns the device status word (0 = healthy); raises
    B200KError if one of the kernels' bounded waits gave up."""
    import ctypes
    lib = _lib.load()
    code = ctypes.c_uint32(0)
    _lib.check(lib.b200k_device_status(_stream(), ctypes.byref(code)))
    return code.value
