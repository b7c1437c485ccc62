"""The example kernels as launchable objects with the reference's call syntax:

    add_kernel[grid](x, y, output, n_elements, BLOCK_SIZE=1024)                  01-vector-add.py:75
    add_kernel_loop[grid](x, y, output, n_elements, row_count, BLOCK_SIZE=1024)  01-vector-add.loop.py:89
    sin_kernel[grid](x, output, n_elements, BLOCK_SIZE=1024)                     01-sin-kernel.py:36
    matmul_kernel_tma[grid](a_desc, b_desc, c_desc, M, N, K, FP8_OUTPUT=..., WARP_SPECIALIZE=...)
                                                                                 09-persistent-matmul.ttnn.py:167-172
    matmul_kernel_fused[grid](a_desc, b_desc, c_desc, bias_desc, M, N, K, ...)   09-matmul-fused.py:175-180
    matmul_kernel[grid](a, b, c, M, N, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0),
                        c.stride(1), ACTIVATION=...)                             03-matrix-multiplication.py:413-420
    _attn_fwd[grid](sm_scale, M, Z, H, desc_q, desc_k, desc_v, desc_o, N_CTX=..., HEAD_DIM=...,
                    FP8_OUTPUT=..., STAGE=..., warp_specialize=..., IS_HOPPER=...) 06-fused-attention.py:257-267

`grid` is a tuple or a callable of the meta-parameters, as in Triton.  A launch goes through the
driver's launcher exactly as a compiled Triton kernel would (driver.py in this package), which
drops the constexpr arguments, flattens descriptors and calls the C-ABI.  The meta-parameters a
grid callable sees are the tile sizes of the hand-written kernels; the grid is validated against
the problem but does not change the result (the kernels are persistent).
"""
from __future__ import annotations

import torch

from . import driver as _driver
from .tensor_descriptor import TensorDescriptor

_IGNORED_LAUNCH_KWARGS = {"num_warps", "num_stages", "num_ctas", "maxnreg", "warmup"}

# launch hooks in the role of triton.compiler.CompiledKernel.launch_enter_hook / launch_exit_hook
launch_enter_hook = None
launch_exit_hook = None


class Kernel:
    def __init__(self, name, arg_names, arg_types, meta_defaults, spec_keys=(), spec_fn=None):
        self.name = name
        self.arg_names = tuple(arg_names)
        self.arg_types = dict(zip(arg_names, arg_types))
        self.meta_defaults = dict(meta_defaults)
        self.spec_keys = tuple(spec_keys)
        self.spec_fn = spec_fn  # extra "KEY=VAL" items derived from the arguments (e.g. the element type)
        self.src = _driver.KernelSource(name=name, arg_names=self.arg_names,
                                        signature={i: self.arg_types[n] for i, n in enumerate(self.arg_names)})
        self.launcher = None
        self.fn = self  # the reference exposes the raw JIT function of an autotuned kernel as `.fn`

    def __getitem__(self, grid):
        return lambda *args, **kwargs: self.run(*args, grid=grid, **kwargs)

    def run(self, *args, grid, **kwargs):
        for k in list(kwargs):
            if k in _IGNORED_LAUNCH_KWARGS:
                kwargs.pop(k)
        if len(args) > len(self.arg_names):
            raise TypeError(f"{self.name}: too many positional arguments")
        bound = dict(zip(self.arg_names, args))
        for k, v in kwargs.items():
            if k not in self.arg_types:
                raise TypeError(f"{self.name}: unexpected argument {k!r}")
            if k in bound:
                raise TypeError(f"{self.name}: argument {k!r} given twice")
            bound[k] = v
        for k, v in self.meta_defaults.items():
            bound.setdefault(k, v)
        missing = [n for n in self.arg_names if n not in bound]
        if missing:
            raise TypeError(f"{self.name}: missing arguments {missing}")
        if bound.get("FP8_OUTPUT"):
            raise NotImplementedError(f"{self.name}: FP8 output is not built")
        for n in self.arg_names:
            v = bound[n]
            t = v.base if isinstance(v, TensorDescriptor) else v
            if isinstance(t, torch.Tensor) and not t.is_cuda:
                raise ValueError(f"{self.name}: argument {n!r} must live on a CUDA device (use the wrappers in "
                                 "triton_tenstorrent_b200.ops for host tensors)")
        meta = {n: bound[n] for n in self.arg_names if self.arg_types[n] == "constexpr"}
        g = grid(meta) if callable(grid) else grid
        g = tuple(g) + (1,) * (3 - len(g))
        items = [f"{k}={int(bound[k])}" for k in self.spec_keys]
        if self.spec_fn is not None:
            items.extend(self.spec_fn(bound))
        spec = ",".join(items)
        function = f"{self.name}:{spec}" if spec else self.name
        drv = _driver.active
        if self.launcher is None:
            drv.utils.load_binary(function, b"", 0, 0)
            self.launcher = drv.launcher_cls(self.src, None)
        stream = drv.get_current_stream()
        self.launcher(g[0], g[1], g[2], stream, function, _driver.pack_metadata(), None, launch_enter_hook,
                      launch_exit_hook, *[bound[n] for n in self.arg_names])


def _add_spec(bound):
    """The element type is a compile-time property of the reference kernel (fp32 in 01-vector-add.py, bf16 in
    01-vector-add.loop.py:102-103); here it travels in the name."""
    dt = bound["x_ptr"].dtype
    if dt != bound["y_ptr"].dtype or dt != bound["output_ptr"].dtype or dt not in (torch.float32, torch.bfloat16):
        raise TypeError("add_kernel: x, y and output must all be fp32 or all bf16")
    return ["BF16=1"] if dt == torch.bfloat16 else []


add_kernel = Kernel(
    "add_kernel", ["x_ptr", "y_ptr", "output_ptr", "n_elements", "BLOCK_SIZE"],
    ["*fp32", "*fp32", "*fp32", "i32", "constexpr"], {}, spec_keys=("BLOCK_SIZE",), spec_fn=_add_spec)

# add_kernel of python/tutorials/01-vector-add.loop.py:29-35: one more scalar, row_count (launch :89)
add_kernel_loop = Kernel(
    "add_kernel", ["x_ptr", "y_ptr", "output_ptr", "n_elements", "row_count", "BLOCK_SIZE"],
    ["*fp32", "*fp32", "*fp32", "i32", "i32", "constexpr"], {}, spec_keys=("BLOCK_SIZE",), spec_fn=_add_spec)

sin_kernel = Kernel(
    "sin_kernel", ["x_ptr", "output_ptr", "n_elements", "BLOCK_SIZE"],
    ["*fp32", "*fp32", "i32", "constexpr"], {}, spec_keys=("BLOCK_SIZE",))

# python/tutorials/gluon/01-intro.py:84-93 (launch :96-99) and :50-53 (launch :60-63)
memcpy_kernel = Kernel(
    "memcpy_kernel", ["in_ptr", "out_ptr", "xnumel", "XBLOCK"], ["*fp32", "*fp32", "i32", "constexpr"], {},
    spec_keys=("XBLOCK",))

copy_scalar_kernel = Kernel("copy_scalar_kernel", ["in_ptr", "out_ptr"], ["*fp32", "*fp32"], {})

mul_add_kernel = Kernel(
    "mul_add_kernel", ["x_ptr", "y_ptr", "z_ptr", "output_ptr", "n_elements", "BLOCK_SIZE"],
    ["*fp32", "*fp32", "*fp32", "*fp32", "i32", "constexpr"], {}, spec_keys=("BLOCK_SIZE",))

def _matmul_spec(bound):
    """The compiled reference kernel is specialised on the descriptors' element type; here it travels in the name."""
    return ["F16=1"] if bound["a_desc"].base.dtype == torch.float16 else []


_MATMUL_META = {"BLOCK_SIZE_M": 128, "BLOCK_SIZE_N": 256, "BLOCK_SIZE_K": 64, "GROUP_SIZE_M": 8,
                "FP8_OUTPUT": False, "WARP_SPECIALIZE": True}

matmul_kernel_tma = Kernel(
    "matmul_kernel_tma",
    ["a_desc", "b_desc", "c_desc", "M", "N", "K", "BLOCK_SIZE_M", "BLOCK_SIZE_N", "BLOCK_SIZE_K", "GROUP_SIZE_M",
     "FP8_OUTPUT", "WARP_SPECIALIZE"],
    ["tensordesc", "tensordesc", "tensordesc", "i32", "i32", "i32"] + ["constexpr"] * 6, _MATMUL_META,
    spec_fn=_matmul_spec)

matmul_kernel_fused = Kernel(
    "matmul_kernel_fused",
    ["a_desc", "b_desc", "c_desc", "bias_desc", "M", "N", "K", "BLOCK_SIZE_M", "BLOCK_SIZE_N", "BLOCK_SIZE_K",
     "GROUP_SIZE_M", "FP8_OUTPUT", "WARP_SPECIALIZE"],
    ["tensordesc"] * 4 + ["i32", "i32", "i32"] + ["constexpr"] * 6, _MATMUL_META, spec_fn=_matmul_spec)

_ACTIVATION_CODES = {"": 0, "none": 0, "relu": 1, "leaky_relu": 2}


def _matmul_ptr_spec(bound):
    """ACTIVATION and the operand type are compile-time properties of the reference kernel; LAYOUT says whether
    the buffers are row-major ("row", the strides apply) or tile-major as the reference kernel addresses them
    ("tile32", the strides are ignored exactly as examples/matmul/03-matrix-multiplication.py:333-386 ignores them)."""
    act = bound["ACTIVATION"]
    if act not in _ACTIVATION_CODES:
        raise ValueError(f"matmul_kernel: unknown ACTIVATION {act!r}")
    layout = bound["LAYOUT"]
    if layout not in ("row", "tile32"):
        raise ValueError(f"matmul_kernel: unknown LAYOUT {layout!r}")
    a, b, c = bound["a_ptr"], bound["b_ptr"], bound["c_ptr"]
    if not (a.dtype == b.dtype == c.dtype) or a.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("matmul_kernel: a, b, c must share one 16-bit float type")
    if layout == "tile32" and not (a.is_contiguous() and b.is_contiguous() and c.is_contiguous()):
        raise ValueError("matmul_kernel: tile-major buffers must be contiguous")
    return [f"ACTIVATION={_ACTIVATION_CODES[act]}", f"F16={1 if a.dtype == torch.float16 else 0}",
            f"TILE32={1 if layout == 'tile32' else 0}"]


matmul_kernel = Kernel(
    "matmul_kernel",
    ["a_ptr", "b_ptr", "c_ptr", "M", "N", "K", "stride_am", "stride_ak", "stride_bk", "stride_bn", "stride_cm",
     "stride_cn", "BLOCK_SIZE_M", "BLOCK_SIZE_N", "BLOCK_SIZE_K", "GROUP_SIZE_M", "ACTIVATION", "LAYOUT"],
    ["*fp16", "*fp16", "*fp16"] + ["i32"] * 9 + ["constexpr"] * 6,
    {"BLOCK_SIZE_M": 128, "BLOCK_SIZE_N": 256, "BLOCK_SIZE_K": 64, "GROUP_SIZE_M": 8, "ACTIVATION": "", "LAYOUT": "row"},
    spec_keys=("BLOCK_SIZE_M", "BLOCK_SIZE_N"), spec_fn=_matmul_ptr_spec)

_attn_fwd = Kernel(
    "_attn_fwd",
    ["sm_scale", "M", "Z", "H", "desc_q", "desc_k", "desc_v", "desc_o", "N_CTX", "HEAD_DIM", "BLOCK_M", "BLOCK_N",
     "FP8_OUTPUT", "STAGE", "warp_specialize", "IS_HOPPER"],
    ["fp32", "*fp32", "i32", "i32", "tensordesc", "tensordesc", "tensordesc", "tensordesc", "i32"] + ["constexpr"] * 7,
    {"BLOCK_M": 128, "BLOCK_N": 128, "FP8_OUTPUT": False, "STAGE": 1, "warp_specialize": True, "IS_HOPPER": False},
    spec_keys=("STAGE", "BLOCK_M"))
_attn_fwd_jit = _attn_fwd.fn
