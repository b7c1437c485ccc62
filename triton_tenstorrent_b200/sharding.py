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

    Each rank allocates its copy with torch, exports the allocation as a CUDA IPC handle (b200k_ipc_export) and maps
    the other ranks' allocations into its own device's context with peer access (b200k_ipc_open); the 88-byte
    handles travel through all_gather_object of the process group.  Needs one process per GPU on one box with
    direct peer access (NVLink / NVSwitch).  The mappings stay until the process exits, so keep `local` alive and
    do not empty torch's allocator cache while other ranks still store into it.
    `remote_blocks()` lists the addresses of this rank's row block inside every other rank's copy.
    `fence()` is the stream-ordered point after which every rank's block has arrived in the local copy: a
    one-element all-reduce on the current stream (it follows this rank's stores in stream order, and completes
    only when every rank has reached it)."""

    def __init__(self, rows: int, N: int, group=None, device=None):
        import torch
        import torch.distributed as dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.rows, self.N = rows, N
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.local = torch.empty((self.world * rows, N), dtype=torch.bfloat16, device=device)
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        lib = _lib.load()
        mine = _lib.IpcHandle()
        # A failure on one rank (IPC not permitted, no peer access) must not leave the others waiting in a collective:
        # every step's outcome is exchanged and all ranks raise together.
        with torch.cuda.device(device):
            problem = ""
            try:
                _lib.check(lib.b200k_ipc_export(self.local.data_ptr(), ctypes.byref(mine)))
            except Exception as e:  # noqa: BLE001
                problem = f"rank {self.rank}: {e}"
            handles = [None] * self.world
            dist.all_gather_object(handles, (bytes(mine), problem), group=group)
            problems = [p for _, p in handles if p]
            if problems:
                raise RuntimeError("GatheredRows: exporting the buffers failed: " + "; ".join(problems))
            self.copy_ptrs = []
            for r, (raw, _) in enumerate(handles):
                if r == self.rank:
                    self.copy_ptrs.append(self.local.data_ptr())
                    continue
                h = _lib.IpcHandle.from_buffer_copy(raw)
                p = ctypes.c_void_p()
                try:
                    _lib.check(lib.b200k_ipc_open(ctypes.byref(h), ctypes.byref(p)))
                except Exception as e:  # noqa: BLE001
                    problem = f"rank {self.rank} opening rank {r}: {e}"
                    break
                self.copy_ptrs.append(p.value)
            outcomes = [None] * self.world
            dist.all_gather_object(outcomes, problem, group=group)
            problems = [p for p in outcomes if p]
            if problems:
                raise RuntimeError("GatheredRows: mapping the peers' buffers failed: " + "; ".join(problems))

    def own_block(self):
        """This rank's rows inside its own copy (a tensor view)."""
        return self.local[self.rank * self.rows:(self.rank + 1) * self.rows]

    def remote_blocks(self):
        """Addresses of this rank's rows inside the other ranks' copies."""
        off = self.rank * self.rows * self.N * 2
        return [p + off for r, p in enumerate(self.copy_ptrs) if r != self.rank]

    def fence(self):
        import torch.distributed as dist
        dist.all_reduce(self._flag, group=self.group)


def matmul_all_gather(a_shard, b, gathered: "GatheredRows", bias=None, activation: str = ""):
    """This rank's rows of C = act(A.B [+ bias]) computed once and stored by the kernel into every rank's copy of
    the full C; returns the local full C, complete after the fence."""
    from . import ops
    ops.matmul_multi(a_shard, b, [gathered.own_block()], bias=bias, activation=activation,
                     remote_ptrs=gathered.remote_blocks())
    gathered.fence()
    return gathered.local


def attention_all_gather(q_shard, k_shard, v_shard, causal, sm_scale, gathered: "GatheredRows"):
    """Attention over this rank's (batch, head) shard ([Zs,Hs,N_CTX,D] with Zs*Hs*N_CTX == gathered.rows and
    D == gathered.N) whose O tiles the kernel stores into every rank's copy of the full O; returns the local full O
    as a [world * rows, D] matrix, complete after the fence."""
    from . import ops
    ops.attention_multi(q_shard, k_shard, v_shard, causal, sm_scale, gathered.own_block(),
                        remote_ptrs=gathered.remote_blocks())
    gathered.fence()
    return gathered.local


def host_b_bytes(b_host, world: int) -> int:
    """Bytes of B this rank uploads in matmul_tma_host_sharded: its 1/world of the rows when K divides evenly
    (the rest arrives over NVLink), else all of B."""
    K = b_host.shape[0]
    rows = K // world if K % world == 0 else K
    return rows * b_host.shape[1] * b_host.element_size()


def matmul_tma_host_sharded(a_shard, b, out_shard=None, group=None):
    """This rank's rows of C = A.B for HOST operands on a box of several GPUs (one process per GPU).

    `a_shard` is the rank's row block of A, `b` the whole of B, both host tensors (pinned for asynchronous
    copies); the result lands in `out_shard` (host).  B crosses the host link once for the whole box: every
    rank uploads K/world of its rows and the ranks all-gather them over NVLink (NCCL), instead of every rank
    uploading all of B.  A's rows then stream to the GPU in row blocks while earlier blocks multiply and
    finished rows of C stream back (ops' host pipeline).  Falls back to uploading all of B when K does not
    divide by the number of ranks."""
    import torch
    import torch.distributed as dist
    from . import ops
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    K, N = b.shape
    device = torch.device("cuda", torch.cuda.current_device())
    if K % world == 0:
        rows = K // world
        b_dev = torch.empty((K, N), dtype=b.dtype, device=device)
        mine = b_dev[rank * rows:(rank + 1) * rows]
        mine.copy_(b[rank * rows:(rank + 1) * rows], non_blocking=True)
        dist.all_gather_into_tensor(b_dev, mine, group=group)
    else:
        b_dev = b.to(device, non_blocking=True)
    return ops.matmul_tma_host_rows(a_shard, b_dev, out_shard)
