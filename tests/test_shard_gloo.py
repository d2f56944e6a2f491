"""CPU tests of the column-split host logic, including a world_size-2 run over
gloo: each rank computes its column block (with the oracle standing in for the
GPU kernel), the blocks are all-gathered shard-major and re-laid out row-major,
and the result must equal the unsharded computation bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from vpipe_b200 import shard, synth


def test_shard_rows_and_fixed_shards():
    assert shard.shard_rows(12288, 4, 1) == (3072, 6144)
    assert shard.shard_rows(13824, 8, 7) == (12096, 13824)     # 1728-wide shards
    with pytest.raises(ValueError):
        shard.shard_rows(100, 8, 0)
    with pytest.raises(ValueError):
        shard.shard_rows(64, 2, 2)
    # a weight fixed at 8 column shards spread over 1 / 2 / 4 / 8 GPUs
    for world in (1, 2, 4, 8):
        cover = []
        for r in range(world):
            cover += shard.fixed_shards(15360, 8, world, r)
        assert cover == [(i * 1920, (i + 1) * 1920) for i in range(8)]
    with pytest.raises(ValueError):
        shard.fixed_shards(15360, 8, 3, 0)


def test_row_slices_are_byte_slices():
    codes, s, b = synth.random_qweight(64, 256, 5)
    lo, hi = shard.shard_rows(64, 4, 2)
    assert shard.take_rows(codes, lo, hi).tobytes() == codes.tobytes()[lo * 128:hi * 128]
    assert shard.take_rows(s, lo, hi).tobytes() == s.tobytes()[lo * 8:hi * 8]


def test_shards_to_rowmajor():
    G, M, ns = 4, 5, 6
    y = np.arange(G * M * ns, dtype=np.int32).reshape(G, M, ns)
    out = shard.shards_to_rowmajor(y)
    for g in range(G):
        assert np.array_equal(out[:, g * ns:(g + 1) * ns], y[g])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, N, K, M, out_dir):
    import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        codes, s, b = synth.random_qweight(N, K, 91)
        x = synth.activations_bf16(M, K, 92)
        lo, hi = shard.shard_rows(N, world, rank)
        y_mine = oracle.qmm_kernel_numerics(shard.take_rows(codes, lo, hi), shard.take_rows(s, lo, hi),
                                            shard.take_rows(b, lo, hi), x, threads=1)
        mine = torch.from_numpy(y_mine.view(np.uint8))   # gloo moves bytes
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        y_shards = torch.stack(parts).numpy().view(np.uint16)          # [G, M, N/G] bf16 bits
        y = shard.shards_to_rowmajor(y_shards)
        full = oracle.qmm_kernel_numerics(codes, s, b, x, threads=1)
        ok = np.array_equal(y, full)
        # a rank with a mismatched shard width must be caught on the host
        try:
            shard.shard_rows(N + 1, world, rank)
            ok = False
        except ValueError:
            pass
        np.save(os.path.join(out_dir, f"ok{rank}.npy"), np.array(ok))
    finally:
        dist.destroy_process_group()


def test_world2_gloo_column_split_equals_unsharded(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), 96, 256, 17, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert bool(np.load(tmp_path / f"ok{r}.npy"))
