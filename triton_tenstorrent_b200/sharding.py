"""Work partition across the GPUs of one box: matmul by M-row blocks of C with B replicated,
attention by (batch, head) pairs.  Every rank runs the single-GPU kernels on its shard; no
collective is needed to produce the shards' results.  `all_gather_rows` is the optional
NCCL all-gather of the output, timed separately by the benchmark.

The split is the reference's contiguous-range formula for distributing blocks over workers
(npu/lib/TritonNPUToTenstorrent/D2M/SPMDOpToD2M.cpp:77-113): base = nb / W, rem = nb % W, worker w
gets [w*base + min(w, rem), ... + base + (w < rem)).
"""
from __future__ import annotations

import ctypes

from . import _lib


def block_range(num_blocks: int, workers: int, w: int):
    """[start, end) of worker `w`; computed by the C-ABI so that host and library agree."""
    s, e = ctypes.c_int64(), ctypes.c_int64()
    _lib.check(_lib.load().b200k_block_range(num_blocks, workers, w, ctypes.byref(s), ctypes.byref(e)))
    return s.value, e.value


def row_shard(M: int, world: int, rank: int, tile: int = 128):
    """Rows [r0, r1) of A and C owned by `rank`: whole 128-row tiles, split by block_range."""
    nb = (M + tile - 1) // tile
    s, e = block_range(nb, world, rank)
    return min(s * tile, M), min(e * tile, M)


def head_shard(ZH: int, world: int, rank: int):
    """(batch*head) indices [h0, h1) owned by `rank`."""
    return block_range(ZH, world, rank)


def all_gather_rows(c_shard, group=None):
    """Gathers equally sized row shards of C from all ranks into one [world*rows, N] tensor
    (torch.distributed all_gather_into_tensor: NCCL over NVLink on GPUs, gloo on CPU tensors)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    out = torch.empty((world * c_shard.shape[0],) + tuple(c_shard.shape[1:]), dtype=c_shard.dtype, device=c_shard.device)
    if c_shard.is_cuda:
        dist.all_gather_into_tensor(out, c_shard.contiguous(), group=group)
    else:
        parts = list(out.chunk(world, dim=0))
        dist.all_gather(parts, c_shard.contiguous(), group=group)
    return out
