"""Seeded inputs shared by the golden-vector generator and the tests.

Every generator draws on the CPU with torch.manual_seed(seed) so that the oracle, the CUDA path and
the golden vectors all see identical bits.  Distributions follow the workload definitions:
add x,y ~ U[0,1); sin x ~ U[-4pi, 4pi); matmul A,B ~ N(0,1)/sqrt(K) in bf16; fused bias; attention
q,k,v ~ N(0,1) in bf16.
"""
from __future__ import annotations

import hashlib
import math

import torch

ADD_SIZES = [1, 33, 1024, 5000, 98432]
SIN_SIZES = [32, 1024, 98432]
MUL_ADD_SIZES = [1, 1000, 4097, 98432]
# (n, programs, row_count) of the row_count-loop add_kernel; the first is the tutorial's own launch
# (n_cores = 130 > 97 rows, so 97 programs of one row each), the last leaves elements uncovered
ADD_LOOP_CASES = [(98432, 97, 1), (50000, 7, 7), (33333, 3, 11), (50000, 5, 7)]
MATMUL_SHAPES = [(32, 32, 32), (64, 32, 32), (128, 256, 64), (96, 160, 136), (256, 256, 256)]
FUSED_SHAPES = [(64, 64, 256), (128, 192, 512)]
# (M, N, K, ACTIVATION) of the pointer-based matmul_kernel on tile-major fp16 buffers
TILE32_CASES = [(32, 32, 64, ""), (64, 96, 128, "leaky_relu"), (128, 256, 96, ""), (256, 128, 256, "leaky_relu")]
# (Z, H, N_CTX, HEAD_DIM, causal, BLOCK_M, BLOCK_N); BLOCK_N <= HEAD_DIM as the reference asserts
ATTN_CASES = [
    (1, 2, 256, 128, False, 128, 128),
    (1, 2, 256, 128, True, 128, 128),
    (1, 1, 384, 128, True, 128, 128),
    (1, 1, 128, 128, True, 32, 32),
    (1, 2, 128, 64, True, 64, 64),
    (1, 2, 128, 16, True, 32, 16),
    (1, 2, 128, 32, False, 64, 32),
    (1, 1, 256, 256, True, 64, 64),
    # sequence lengths that are multiples of the reference's smaller blocks but not of 128
    (1, 2, 192, 128, True, 64, 64),
    (1, 2, 320, 64, False, 64, 64),
    (1, 1, 96, 32, True, 32, 32),
]


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def add_inputs(n: int, seed: int = 0):
    g = _gen(seed)
    return torch.rand(n, generator=g, dtype=torch.float32), torch.rand(n, generator=g, dtype=torch.float32)


def mul_add_inputs(n: int, seed: int = 7):
    """x, y ~ U[0,1) and z ~ U[-4pi, 4pi): products and sums that round (x*y is rounded before z is added)."""
    g = _gen(seed)
    x = torch.rand(n, generator=g, dtype=torch.float32)
    y = torch.rand(n, generator=g, dtype=torch.float32)
    z = (torch.rand(n, generator=g, dtype=torch.float32) * 8 - 4) * math.pi
    return x, y, z


def sin_inputs(n: int, seed: int = 0):
    g = _gen(seed)
    return (torch.rand(n, generator=g, dtype=torch.float32) * 8 - 4) * math.pi


def matmul_inputs(M: int, N: int, K: int, seed: int = 0, dtype=torch.bfloat16):
    g = _gen(seed)
    a = (torch.randn(M, K, generator=g, dtype=torch.float32) / math.sqrt(K)).to(dtype)
    b = (torch.randn(K, N, generator=g, dtype=torch.float32) / math.sqrt(K)).to(dtype)
    return a, b


def fused_inputs(M: int, N: int, K: int, seed: int = 0, dtype=torch.bfloat16):
    """A, B as matmul_inputs plus the reference's full [M,N] bias in the operand dtype."""
    g = _gen(seed)
    a = (torch.randn(M, K, generator=g, dtype=torch.float32) / math.sqrt(K)).to(dtype)
    b = (torch.randn(K, N, generator=g, dtype=torch.float32) / math.sqrt(K)).to(dtype)
    bias = (torch.randn(M, N, generator=g, dtype=torch.float32) * 0.1).to(dtype)
    return a, b, bias


def tile32_inputs(M: int, N: int, K: int, seed: int = 0, dtype=torch.float16):
    """Row-major A, B ~ U[-0.5, 0.5) in fp16, the distribution of the reference's own check of
    matmul_kernel (examples/matmul/03-matrix-multiplication.py:431-432)."""
    g = _gen(seed)
    a = (torch.rand(M, K, generator=g, dtype=torch.float32) - 0.5).to(dtype)
    b = (torch.rand(K, N, generator=g, dtype=torch.float32) - 0.5).to(dtype)
    return a, b


def tilize(t: torch.Tensor, tile: int = 32) -> torch.Tensor:
    """Row-major [R,S] -> same shape, memory holding contiguous tile x tile tiles in row-major tile order."""
    R, S = t.shape
    return t.reshape(R // tile, tile, S // tile, tile).permute(0, 2, 1, 3).contiguous().view(R, S)


def untilize(t: torch.Tensor, tile: int = 32) -> torch.Tensor:
    R, S = t.shape
    return t.reshape(R // tile, S // tile, tile, tile).permute(0, 2, 1, 3).contiguous().view(R, S)


def row_bias(N: int, seed: int = 1):
    """bias[N] fp32 ~ N(0, 0.1) of the fused-matmul workload."""
    g = _gen(seed)
    return torch.randn(N, generator=g, dtype=torch.float32) * 0.1


def attn_inputs(Z: int, H: int, S: int, D: int, seed: int = 0):
    g = _gen(seed)
    q = torch.randn(Z, H, S, D, generator=g, dtype=torch.float32).bfloat16()
    k = torch.randn(Z, H, S, D, generator=g, dtype=torch.float32).bfloat16()
    v = torch.randn(Z, H, S, D, generator=g, dtype=torch.float32).bfloat16()
    return q, k, v


def digest(*tensors) -> str:
    """sha256 over the raw bytes of the tensors, to detect a drift of the input generators."""
    h = hashlib.sha256()
    for t in tensors:
        t = t.contiguous()
        if t.dtype in (torch.bfloat16, torch.float16):
            t = t.view(torch.int16)
        h.update(t.numpy().tobytes())
    return h.hexdigest()
