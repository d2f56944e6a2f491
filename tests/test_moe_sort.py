"""Host-side routing sort for the grouped GEMMs (vpipe_b200/moe.py): the bookkeeping of the
reference's moe_hist_i32 / moe_sort_setup_i32 / moe_scatter_i32 (ops/llm_elementwise.metal:252-325)."""
import numpy as np
import pytest

from vpipe_b200 import moe


def test_sort_pairs_small_case_by_hand():
    eid = np.array([2, 0, 2, 2, 0, 3], np.int32)  # 3 tokens x top-2; expert 1 idle
    tile2e, srow, sdst, npad = moe.sort_pairs(eid, 4, 2, 2)
    assert npad == 2 + 4 + 2 and list(tile2e) == [0, 2, 2, 3]
    assert list(sdst) == [1, 4, 0, 2, 3, -1, 5, -1]
    assert list(srow) == [0, 2, 0, 1, 1, -1, 2, -1]


@pytest.mark.parametrize("T,E,top_k,tile", [(1, 1, 1, 128), (257, 16, 4, 128), (1000, 128, 8, 32)])
def test_sort_pairs_properties(T, E, top_k, tile):
    rng = np.random.default_rng(T + E)
    eid = rng.integers(0, E, T * top_k).astype(np.int32)
    tile2e, srow, sdst, npad = moe.sort_pairs(eid, E, top_k, tile)
    assert npad % tile == 0 and tile2e.size == npad // tile
    live = sdst >= 0
    assert sorted(sdst[live]) == list(range(T * top_k))          # every pair exactly once
    assert np.array_equal(srow[live], sdst[live] // top_k)       # its token row
    assert np.all((srow < 0) == ~live)
    slot_e = np.repeat(tile2e, tile)
    assert np.array_equal(slot_e[live], eid[sdst[live]])         # in its own expert's block
    assert np.all(np.diff(tile2e) >= 0)                          # blocks in expert order
    # padding per expert is less than one tile
    for e in np.unique(tile2e):
        assert (slot_e == e).sum() - (eid == e).sum() < tile


def test_sort_pairs_rejects_bad_ids():
    with pytest.raises(ValueError):
        moe.sort_pairs(np.array([0, 5], np.int32), 4, 1, 128)
