"""B200-native implementation of the kernels that kernelize-ai/triton-tenstorrent's examples compile
and run: hand-written sm_100a CUDA behind a C-ABI (include/b200k.h), reached through the examples'
own launch surface.  Importing the package does not load the library; the first call does, and fails
loudly if it has not been built (`python -m triton_tenstorrent_b200.build`)."""
from .ops import (add, add_loop, attention, attention_with_lse, device_status, matmul, matmul_fused, matmul_tma,
                  matmul_tma_fused, memcpy, mul_add, sin, tilize, untilize)
from .tensor_descriptor import TensorDescriptor
from .kernels import (_attn_fwd, _attn_fwd_jit, add_kernel, add_kernel_loop, matmul_kernel, matmul_kernel_fused, matmul_kernel_tma, memcpy_kernel, copy_scalar_kernel,
                      mul_add_kernel, sin_kernel)

__all__ = ["add", "add_loop", "sin", "memcpy", "mul_add", "memcpy_kernel", "copy_scalar_kernel", "matmul", "matmul_tma", "matmul_fused", "matmul_tma_fused", "attention",
           "attention_with_lse", "device_status", "tilize", "untilize", "TensorDescriptor", "add_kernel", "add_kernel_loop", "matmul_kernel", "sin_kernel", "mul_add_kernel",
           "matmul_kernel_tma", "matmul_kernel_fused", "_attn_fwd", "_attn_fwd_jit"]
