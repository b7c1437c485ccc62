"""world_size-2 check of the multi-GPU host logic on CPU (gloo): each rank takes its M-row shard
of A / its (batch, head) shard of q,k,v from the partition helpers, computes it (here with the CPU
oracle standing in for the device), and the optional all-gather of C reassembles the full result.
The path has no data-path collective; the all-gather is the separately timed extra."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import golden_inputs as gi
from oracle import cpu_oracle as oracle
from triton_tenstorrent_b200 import sharding


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ok):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        M, N, K = 512, 256, 128
        a, b = gi.matmul_inputs(M, N, K)                 # same seed on every rank: B is replicated
        r0, r1 = sharding.row_shard(M, world, rank)
        c_shard = oracle.golden_matmul(a[r0:r1], b)
        c = sharding.all_gather_rows(c_shard)
        full = oracle.golden_matmul(a, b)
        assert torch.equal(c.view(torch.int16), full.view(torch.int16))

        Z, H, S, D = 1, 4, 128, 128
        q, k, v = gi.attn_inputs(Z, H, S, D)
        h0, h1 = sharding.head_shard(Z * H, world, rank)
        qs, ks, vs = (t.reshape(Z * H, S, D)[h0:h1].reshape(1, h1 - h0, S, D) for t in (q, k, v))
        o_shard, _ = oracle.attention(qs, ks, vs, True, D ** -0.5)
        o_full, _ = oracle.attention(q, k, v, True, D ** -0.5)
        assert torch.equal(o_shard.view(torch.int16).reshape(-1, S, D),
                           o_full.view(torch.int16).reshape(Z * H, S, D)[h0:h1])
        dist.barrier()
        ok[rank] = 1
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_and_gather():
    world = 2
    ctx = mp.get_context("spawn")
    ok = ctx.Array("i", [0] * world)
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ok)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert list(ok) == [1] * world
