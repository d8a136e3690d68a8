"""Index math of the persistent GEMM tile order, evaluated on the host by the same function the
kernels run: every tile exactly once; the rank pivot puts the intended slab first and the own
slab last (reduce-scatter) or the local shard first (all-gather); groups never straddle slabs."""
import ctypes

import pytest

from kraken_b200.ops import lib as klib


def _order(tiles_r, tiles_c, group_r, pivot_r, interleave_r=0):
    buf = (ctypes.c_int * (2 * tiles_r * tiles_c))()
    klib.check(klib.lib().kr_tile_order(tiles_r, tiles_c, group_r, pivot_r, interleave_r, buf))
    return [(buf[2 * i], buf[2 * i + 1]) for i in range(tiles_r * tiles_c)]


@pytest.mark.parametrize("tiles_r,tiles_c,group_r,pivot_r", [(1, 1, 1, 0), (7, 5, 3, 0), (64, 112, 16, 0), (32, 32, 4, 12),
                                                             (9, 4, 16, 8), (16, 3, 8, 15)])
def test_every_tile_exactly_once(tiles_r, tiles_c, group_r, pivot_r):
    order = _order(tiles_r, tiles_c, group_r, pivot_r)
    assert sorted(order) == [(r, c) for r in range(tiles_r) for c in range(tiles_c)]


@pytest.mark.parametrize("ws,rank", [(2, 0), (2, 1), (4, 2), (8, 0), (8, 7), (8, 3)])
def test_reduce_scatter_order_next_ranks_slab_first_own_slab_last(ws, rank):
    tiles_per_slab, tiles_c = 4, 6
    tiles_r = ws * tiles_per_slab
    pivot = (((rank + 1) % ws) * tiles_per_slab) % tiles_r
    order = _order(tiles_r, tiles_c, 4, pivot)
    owners = [r // tiles_per_slab for r, _ in order]
    per_slab = tiles_per_slab * tiles_c
    for i in range(ws):                      # slabs are visited one after another, each completely
        chunk = owners[i * per_slab:(i + 1) * per_slab]
        assert set(chunk) == {(rank + 1 + i) % ws}
    assert owners[-1] == rank


@pytest.mark.parametrize("ws,rank", [(2, 1), (4, 3), (8, 5)])
def test_all_gather_order_starts_on_the_local_shard(ws, rank):
    tiles_per_shard, tiles_c = 8, 3
    tiles_r = ws * tiles_per_shard
    order = _order(tiles_r, tiles_c, 8, rank * tiles_per_shard)
    first = order[: tiles_per_shard * tiles_c]
    assert {r // tiles_per_shard for r, _ in first} == {rank}
    # then the shards in the order the all-gather delivers them: rank+1, rank+2, ...
    nxt = order[tiles_per_shard * tiles_c: 2 * tiles_per_shard * tiles_c]
    assert {r // tiles_per_shard for r, _ in nxt} == {(rank + 1) % ws}


@pytest.mark.parametrize("tiles_r,tiles_c,group_r,il", [(8, 3, 8, 8), (32, 32, 8, 8), (32, 5, 8, 4), (16, 7, 8, 2), (12, 4, 8, 3)])
def test_interleaved_slabs_every_tile_once_and_owners_rotate(tiles_r, tiles_c, group_r, il):
    order = _order(tiles_r, tiles_c, group_r, 0, il)
    assert sorted(order) == [(r, c) for r in range(tiles_r) for c in range(tiles_c)]
    per_slab = tiles_r // il
    # the first `il` tiles of the order hit `il` different slabs when a group holds at least `il` rows
    if group_r >= il:
        assert {r // per_slab for r, _ in order[:il]} == set(range(il))


@pytest.mark.parametrize("ws,rank,T,C", [(8, 3, 4, 1), (8, 0, 4, 2), (4, 3, 8, 2), (2, 1, 16, 4), (3, 2, 6, 3), (1, 0, 4, 2)])
def test_all_gather_chunk_major_order(ws, rank, T, C):
    # multicast push: own shard first, then chunk 0 of every peer (rank+1, rank+2, ...), chunk 1 of every peer, ...
    tiles_c = 5
    n = ws * T * tiles_c
    buf = (ctypes.c_int * (2 * n))()
    klib.check(klib.lib().kr_tile_order_ag(tiles_c, C, rank, ws, T, C, buf))
    order = [(buf[2 * i], buf[2 * i + 1]) for i in range(n)]
    assert sorted(order) == [(r, c) for r in range(ws * T) for c in range(tiles_c)]
    rows = []
    for r, _ in order:                       # row tiles in order of first appearance
        if r not in rows:
            rows.append(r)
    expect = [rank * T + i for i in range(T)]
    for c in range(T // C):
        for s in range(1, ws):
            src = (rank + s) % ws
            expect += [src * T + c * C + t for t in range(C)]
    assert rows == expect
