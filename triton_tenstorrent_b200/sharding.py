"""Work partition across the GPUs of one box: matmul by M-row blocks of C with B replicated,
attention by (batch, head) pairs.  Every rank runs the single-GPU kernels on its shard; no
collective is needed to produce the shards' results.  `all_gather_rows` is the optional
NCCL all-gather of the output, timed separately by the benchmark; `GatheredRows` does the same
gather inside the matmul kernel (its epilogue stores every tile into all GPUs' copies of C).

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


class GatheredRows:
    """A full [world * rows, N] bf16 matrix on every rank whose copies are all mapped into every rank's process,
    so that one rank's matmul epilogue can store its row block into all of them (ops.matmul_multi).

    Each rank allocates its copy with torch, exports it as a CUDA IPC handle
    (torch.multiprocessing.reductions.reduce_tensor) and opens the other ranks' handles; the handles travel
    through all_gather_object of the process group.  Needs one process per GPU on one box with peer access
    (NVLink / NVSwitch).  `dests()` lists, own copy first, the views of this rank's row block in every copy.
    `fence()` is the stream-ordered point after which every rank's block has arrived in the local copy: a
    one-element all-reduce on the current stream (it follows this rank's stores in stream order, and completes
    only when every rank has reached it)."""

    def __init__(self, rows: int, N: int, group=None, device=None):
        import torch
        import torch.distributed as dist
        from torch.multiprocessing.reductions import reduce_tensor
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.rows, self.N = rows, N
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.local = torch.empty((self.world * rows, N), dtype=torch.bfloat16, device=device)
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        handles = [None] * self.world
        dist.all_gather_object(handles, reduce_tensor(self.local), group=group)
        with torch.cuda.device(device):   # peer access is enabled for the device current while a handle is opened
            self.copies = [self.local if r == self.rank else fn(*args) for r, (fn, args) in enumerate(handles)]
        for r, c in enumerate(self.copies):
            if tuple(c.shape) != tuple(self.local.shape) or c.dtype != self.local.dtype:
                raise RuntimeError(f"rank {r} exported a {tuple(c.shape)} {c.dtype} buffer")

    def block(self, copy_rank: int, block_rank: int):
        """Rows of `block_rank` inside rank `copy_rank`'s copy."""
        return self.copies[copy_rank][block_rank * self.rows:(block_rank + 1) * self.rows]

    def dests(self):
        order = [self.rank] + [r for r in range(self.world) if r != self.rank]
        return [self.block(r, self.rank) for r in order]

    def fence(self):
        import torch.distributed as dist
        dist.all_reduce(self._flag, group=self.group)


def matmul_all_gather(a_shard, b, gathered: "GatheredRows", bias=None, activation: str = ""):
    """This rank's rows of C = act(A.B [+ bias]) computed once and stored by the kernel into every rank's copy of
    the full C; returns the local full C, complete after the fence."""
    from . import ops
    ops.matmul_multi(a_shard, b, gathered.dests(), bias=bias, activation=activation)
    gathered.fence()
    return gathered.local
