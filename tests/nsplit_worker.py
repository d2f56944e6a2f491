"""Worker of the multi-GPU column-split test (launched by torch.distributed.run, one rank per GPU).

Every rank quantizes the same seeded weight on its GPU, keeps its row shard, runs the sharded QMM
with the NCCL gather through the C ABI, and compares the gathered result (shard-major and
row-major) with the unsharded QMM run locally. Exit code 0 on success."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from vpipe_b200 import ops, shard


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    comm = shard.NsplitComm(rank, world, dev)
    ok = True
    for (M, K, N, chunks) in [(512, 1024, 1024, 1), (1000, 2048, 2048 * world // 2, 3), (4096, 4096, 12288, 4)]:
        g = torch.Generator(device=dev).manual_seed(1234 + N)
        w = (torch.randn((N, K), generator=g, device=dev) * 0.02).to(torch.bfloat16)
        x = torch.randn((M, K), generator=g, device=dev).to(torch.bfloat16)
        codes, s16, b16 = ops.quantize(w)
        s, b = ops.scales_to_bf16(s16), ops.scales_to_bf16(b16)
        full = ops.qmm(codes, s, b, x)
        lo, hi = shard.shard_rows(N, world, rank)
        cs, ss, bs = codes[lo:hi].contiguous(), s[lo:hi].contiguous(), b[lo:hi].contiguous()
        y_shards = torch.zeros((world, M, N // world), dtype=torch.bfloat16, device=dev)
        y_row = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
        comm.qmm(cs, ss, bs, x, y_shards, y_row, m_chunks=chunks)
        torch.cuda.synchronize()
        ref_shards = torch.stack([full[:, r * (N // world):(r + 1) * (N // world)] for r in range(world)])
        good = torch.equal(y_shards, ref_shards) and torch.equal(y_row, full)
        ok = ok and good
        if rank == 0:
            print(f"nsplit world={world} M={M} K={K} N={N} chunks={chunks}: {'ok' if good else 'MISMATCH'}", flush=True)
    # fused form: no collective; every rank's epilogue stores into every rank's row-major y
    for (M, K, N) in [(512, 1024, 1024), (1000, 2048, 2048), (4096, 4096, 12288)]:
        g = torch.Generator(device=dev).manual_seed(4321 + N)
        w = (torch.randn((N, K), generator=g, device=dev) * 0.02).to(torch.bfloat16)
        x = torch.randn((M, K), generator=g, device=dev).to(torch.bfloat16)
        codes, s16, b16 = ops.quantize(w)
        s, b = ops.scales_to_bf16(s16), ops.scales_to_bf16(b16)
        full = ops.qmm(codes, s, b, x)
        lo, hi = shard.shard_rows(N, world, rank)
        cs, ss, bs = codes[lo:hi].contiguous(), s[lo:hi].contiguous(), b[lo:hi].contiguous()
        y_sym, y_ptr = comm.alloc_symmetric((M, N), torch.bfloat16)
        good = True
        for _ in range(2):      # twice: the barrier epoch advances
            y_sym.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            comm.qmm_fused(cs, ss, bs, x, y_ptr)
            torch.cuda.synchronize()
            good = good and torch.equal(y_sym, full)
        ok = ok and good
        if rank == 0:
            print(f"nsplit-fused world={world} M={M} K={K} N={N}: {'ok' if good else 'MISMATCH'}", flush=True)
    # Back-to-back fused calls into ONE symmetric buffer with no host synchronisation: each result is
    # consumed on the stream (copied aside) before the next call; the entry barrier of the next call
    # must keep a fast rank from overwriting y under a slow rank's copy.
    M, K, N = 2048, 2048, 4096
    g = torch.Generator(device=dev).manual_seed(777)
    w = (torch.randn((N, K), generator=g, device=dev) * 0.02).to(torch.bfloat16)
    xs = [torch.randn((M, K), generator=g, device=dev).to(torch.bfloat16) for _ in range(2)]
    codes, s16, b16 = ops.quantize(w)
    s, b = ops.scales_to_bf16(s16), ops.scales_to_bf16(b16)
    fulls = [ops.qmm(codes, s, b, x) for x in xs]
    lo, hi = shard.shard_rows(N, world, rank)
    cs, ss, bs = codes[lo:hi].contiguous(), s[lo:hi].contiguous(), b[lo:hi].contiguous()
    y_sym, y_ptr = comm.alloc_symmetric((M, N), torch.bfloat16)
    keep = [torch.empty_like(y_sym) for _ in range(6)]
    torch.cuda.synchronize()
    dist.barrier()
    for i in range(6):
        comm.qmm_fused(cs, ss, bs, xs[i % 2], y_ptr)
        keep[i].copy_(y_sym)
        if rank == i % world:      # one rank lags behind in every step
            torch.cuda._sleep(2_000_000)
    torch.cuda.synchronize()
    good = all(torch.equal(keep[i], fulls[i % 2]) for i in range(6))
    ok = ok and good
    if rank == 0:
        print(f"nsplit-fused back-to-back world={world}: {'ok' if good else 'MISMATCH'}", flush=True)
    assert ops.device_status() == 0
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    comm.close()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
