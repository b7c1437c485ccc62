"""One rank of the multi-GPU parity check (launched by test_multi_gpu.py through torch.distributed.run, one
process per GPU): the matmul whose epilogue stores this rank's rows of C into every rank's copy of the full
matrix must give, on every rank, exactly what the plain matmul followed by an NCCL all-gather gives."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from triton_tenstorrent_b200 import ops, sharding  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    ok = True
    for (rows, N, K, with_bias) in ((256, 512, 320, False), (1024, 2048, 1024, True), (1152, 4096, 2048, False)):
        g = torch.Generator(device="cpu").manual_seed(100 + rank)
        a = (torch.randn(rows, K, generator=g) / K ** 0.5).bfloat16().cuda()
        gb = torch.Generator(device="cpu").manual_seed(7)
        b = (torch.randn(K, N, generator=gb) / K ** 0.5).bfloat16().cuda()
        bias = (torch.randn(N, generator=gb) * 0.1).cuda() if with_bias else None
        act = "relu" if with_bias else ""
        gathered = sharding.GatheredRows(rows, N)
        print(f"rank {rank}: {len(gathered.remote_blocks())} remote copies mapped", flush=True)
        gathered.local.fill_(7.5)                      # sentinel: every row block must be overwritten
        torch.cuda.synchronize()
        dist.barrier()                                 # nobody stores into a copy that is still being filled
        full = sharding.matmul_all_gather(a, b, gathered, bias=bias, activation=act)
        torch.cuda.synchronize()
        if with_bias:
            own = ops.matmul_fused(a, b, bias, act)
        else:
            own = ops.matmul_tma(a, b)
        ref = sharding.all_gather_rows(own)
        torch.cuda.synchronize()
        same = torch.equal(full.view(torch.int16), ref.view(torch.int16))
        print(f"rank {rank}: rows={rows} N={N} K={K} bias={with_bias} bit-equal={same}", flush=True)
        ok = ok and same
        dist.barrier()
        del gathered
    # attention sharded by (batch, head): every rank's heads, O gathered by the kernel's epilogue
    for (Hs, S, D, causal) in ((2, 256, 128, True), (3, 512, 64, False)):
        g = torch.Generator(device="cpu").manual_seed(200 + rank)
        q, k, v = (torch.randn(1, Hs, S, D, generator=g).bfloat16().cuda() for _ in range(3))
        gathered = sharding.GatheredRows(Hs * S, D)
        gathered.local.fill_(7.5)
        torch.cuda.synchronize()
        dist.barrier()
        full = sharding.attention_all_gather(q, k, v, causal, D ** -0.5, gathered)
        torch.cuda.synchronize()
        ref = sharding.all_gather_rows(ops.attention(q, k, v, causal, D ** -0.5).reshape(Hs * S, D))
        torch.cuda.synchronize()
        same = torch.equal(full.view(torch.int16), ref.view(torch.int16))
        print(f"rank {rank}: attention heads={Hs} S={S} D={D} causal={causal} bit-equal={same}", flush=True)
        ok = ok and same
        dist.barrier()
        del gathered
    status = ops.device_status()
    ok = ok and status == 0
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("MULTI_GPU_PARITY " + ("OK" if int(flag.item()) == 1 else "FAILED"), flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
