"""Column-split of a quantized linear over the GPUs of one box (host logic).

Output columns are rows of W: rank r of G owns rows [r*N/G, (r+1)*N/G) of the
packed weight, the scales and the biases; all three are row-contiguous, so a
shard is a byte slice. x is replicated and the ranks' output column blocks are
all-gathered. The reference is single-GPU; it uses the same row-contiguity to
concatenate q|k|v (generative-models/qwen3/metal-qwen-model.cc:214-250).
"""
from __future__ import annotations

import ctypes as C

import numpy as np


def shard_rows(N: int, world: int, rank: int) -> tuple[int, int]:
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    if N % world:
        raise ValueError(f"N={N} is not a multiple of the {world} ranks")
    ns = N // world
    return rank * ns, (rank + 1) * ns


def fixed_shards(N: int, parts: int, world: int, rank: int) -> list[tuple[int, int]]:
    """A weight cut into `parts` column shards spread over `world` GPUs: rank r
    owns parts/world consecutive shards (all of them when world == 1)."""
    if parts % world:
        raise ValueError(f"{parts} shards do not spread evenly over {world} GPUs")
    if N % parts:
        raise ValueError(f"N={N} is not a multiple of {parts} shards")
    per = parts // world
    w = N // parts
    return [((rank * per + i) * w, (rank * per + i + 1) * w) for i in range(per)]


def take_rows(a, lo: int, hi: int):
    """Rows [lo, hi) of codes / scales / biases (numpy array or torch tensor)."""
    return a[lo:hi]


def shards_to_rowmajor(y_shards: np.ndarray) -> np.ndarray:
    """[G, M, N/G] shard-major -> [M, N] row-major (what the device re-layout does)."""
    G, M, ns = y_shards.shape
    return np.ascontiguousarray(np.transpose(y_shards, (1, 0, 2)).reshape(M, G * ns))


class NsplitComm:
    """NCCL communicator of the C ABI; the unique id travels over torch.distributed."""

    def __init__(self, rank: int, world: int, device=None):
        import torch
        import torch.distributed as dist

        from ._lib import UNIQUE_ID_BYTES, check, lib
        self.rank, self.world = rank, world
        ident = torch.zeros(UNIQUE_ID_BYTES, dtype=torch.uint8)
        if rank == 0:
            buf = (C.c_ubyte * UNIQUE_ID_BYTES)()
            check(lib().vpq_comm_unique_id(buf))
            ident = torch.tensor(list(buf), dtype=torch.uint8)
        if world > 1:
            if dist.get_backend() == "nccl":
                dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
                t = ident.to(dev)
                dist.broadcast(t, src=0)
                ident = t.cpu()
            else:
                dist.broadcast(ident, src=0)
        raw = (C.c_ubyte * UNIQUE_ID_BYTES)(*ident.tolist())
        handle = C.c_void_p()
        check(lib().vpq_comm_create(raw, rank, world, C.byref(handle)))
        self.handle = handle

    def qmm(self, codes_shard, scales_shard, biases_shard, x, y_shards, y_rowmajor=None,
            m_chunks: int = 1, stream=None):
        import torch

        from ._lib import check, lib
        ns, kw = codes_shard.shape
        K = kw * 8
        N = ns * self.world
        M = x.numel() // K
        st = (stream if stream is not None else torch.cuda.current_stream()).cuda_stream
        check(lib().vpq_affine_qmm_w4g64_bf16_nsplit(
            self.handle, codes_shard.data_ptr(), scales_shard.data_ptr(), biases_shard.data_ptr(),
            x.data_ptr(), y_shards.data_ptr(),
            y_rowmajor.data_ptr() if y_rowmajor is not None else None, K, N, M, m_chunks, st))

    def alloc_symmetric(self, shape, dtype):
        """A tensor in a buffer every rank has mapped (collective call). Keep the returned tensor's
        owner (this communicator) alive while it is in use."""
        import torch

        from ._lib import check, lib
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        ptr = C.c_void_p()
        check(lib().vpq_comm_alloc_symmetric(self.handle, nbytes, C.byref(ptr)))

        class _Raw:  # exposes the device allocation through the CUDA array interface
            pass
        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr.value, False),
                                        "version": 2}
        t = torch.as_tensor(raw, device=torch.device("cuda", torch.cuda.current_device()))
        return t.view(dtype).view(*shape), ptr.value

    def free_symmetric(self, ptr) -> None:
        """Releases a buffer of alloc_symmetric (collective: every rank, same order)."""
        from ._lib import check, lib
        check(lib().vpq_comm_free_symmetric(self.handle, ptr))

    def qmm_fused(self, codes_shard, scales_shard, biases_shard, x, y_sym_ptr, stream=None):
        """Column-split QMM whose epilogue writes every rank's row-major y directly (no collective)."""
        import torch

        from ._lib import check, lib
        ns, kw = codes_shard.shape
        K = kw * 8
        N = ns * self.world
        M = x.numel() // K
        st = (stream if stream is not None else torch.cuda.current_stream()).cuda_stream
        check(lib().vpq_affine_qmm_w4g64_bf16_nsplit_fused(
            self.handle, codes_shard.data_ptr(), scales_shard.data_ptr(), biases_shard.data_ptr(),
            x.data_ptr(), y_sym_ptr, K, N, M, st))

    def close(self):
        from ._lib import lib
        if self.handle:
            lib().vpq_comm_destroy(self.handle)
            self.handle = None
