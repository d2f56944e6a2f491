"""Host-side routing sort for the grouped (mixture-of-experts) GEMMs.

The reference sorts (token, expert) pairs into per-expert blocks padded to its row tile with four
small kernels -- histogram, offsets + tile -> expert map, scatter of slots
(gpu-kernels/metal/ops/llm_elementwise.metal:252-325: moe_hist_i32, moe_sort_setup_i32,
moe_scatter_i32) -- and hands the GEMMs three int arrays. This is the same bookkeeping in numpy,
padded to this library's row tile (vpq_qmm_grouped_tile_rows); the order inside an expert's block is
the pair order (the reference leaves it arbitrary)."""
from __future__ import annotations

import numpy as np


def sort_pairs(eid: np.ndarray, experts: int, top_k: int, tile_rows: int):
    """eid [n_pairs]: expert of pair p (pair p belongs to token p // top_k).
    Returns (tile2e [npad / tile_rows], srow [npad], sdst [npad], npad): expert per row tile,
    token row per sorted slot, pair index per sorted slot; padding slots hold -1."""
    eid = np.asarray(eid, np.int64)
    if eid.ndim != 1 or (eid < 0).any() or (eid >= experts).any():
        raise ValueError("sort_pairs: expert ids must be a vector of values in [0, experts)")
    hist = np.bincount(eid, minlength=experts)
    ntile = (hist + tile_rows - 1) // tile_rows
    boff = np.concatenate([[0], np.cumsum(ntile * tile_rows)])
    npad = int(boff[-1])
    tile2e = np.repeat(np.arange(experts, dtype=np.int32), ntile).astype(np.int32)
    srow = np.full(npad, -1, np.int32)
    sdst = np.full(npad, -1, np.int32)
    order = np.argsort(eid, kind="stable")
    rank = np.arange(eid.size) - np.repeat(np.concatenate([[0], np.cumsum(hist)[:-1]]), hist)
    slots = boff[eid[order]] + rank
    srow[slots] = (order // top_k).astype(np.int32)
    sdst[slots] = order.astype(np.int32)
    return tile2e, srow, sdst, npad
