"""Host model of the flag protocol of the fused GEMM -> reduce-scatter kernels, driven by the
launcher's own tiling plan (``kr_rs_plan``) and the tile order the kernels run (``kr_tile_order``).

Every worker (a CTA, or a CTA pair) of every rank walks its tiles in order. The rules modelled:

push   a remote tile's signal to its owner is sent one tile late (the TMA-store epilogue defers
       the completion hook); an own-slab tile first waits for ws-1 signals from the peers. With
       ``flush_before_wait`` the held-back signal is sent before any wait, as the kernels do.
pull   (and scatter) no epilogue ever waits; every tile (own ones too) signals its owner, one tile
       late; each owned tile is cut into work items dealt round-robin to the owner's CTAs, whose
       reducer warps wait for the tile's ws signals.

The model runs to a fixed point; a worker that can never advance is a deadlock. The cases include
the shapes of the tensor-parallel MLP benchmark (M 2048 and 8192, N 8192) at 2, 4 and 8 ranks on 74
CTA pairs and on 148 single CTAs.
"""
import ctypes

import pytest

from kraken_b200.ops import lib as klib


def _plan(M, N, ws, rank, algo, ctas, pair):
    out = (ctypes.c_int * 9)()
    klib.check(klib.lib().kr_rs_plan(M, N, ws, rank, algo, ctas, 1 if pair else 0, out))
    keys = ["pair", "tiles_r", "tiles_c", "group_r", "pivot_r", "interleave_r", "workers", "grid", "sub_rows"]
    return dict(zip(keys, list(out)))


def _order(pl):
    n = pl["tiles_r"] * pl["tiles_c"]
    buf = (ctypes.c_int * (2 * n))()
    klib.check(klib.lib().kr_tile_order(pl["tiles_r"], pl["tiles_c"], pl["group_r"], pl["pivot_r"],
                                        pl["interleave_r"], buf))
    return [(buf[2 * i], buf[2 * i + 1]) for i in range(n)]


def simulate_push(M, N, ws, ctas, pair, flush_before_wait):
    """Returns the number of workers (over all ranks) that never finish."""
    plans = [_plan(M, N, ws, r, 0, ctas, pair) for r in range(ws)]
    orders = [_order(pl) for pl in plans]
    rows_per_tile = 256 if plans[0]["pair"] else 128
    slab_tiles = (M // ws) // rows_per_tile
    W = plans[0]["workers"]
    seqs = {(r, w): orders[r][w::W] for r in range(ws) for w in range(W)}
    pos = {k: 0 for k in seqs}
    held = {k: None for k in seqs}            # tile whose signal is still held back
    flags = {}                                # (owner, tile) -> signals received
    progress = True
    while progress:
        progress = False
        for (r, w), seq in seqs.items():
            while True:
                i = pos[(r, w)]
                if i == len(seq):
                    if held[(r, w)] is not None:
                        o, t = held[(r, w)]
                        flags[(o, t)] = flags.get((o, t), 0) + 1
                        held[(r, w)] = None
                        progress = True
                    break
                tr, tc = seq[i]
                owner = tr // slab_tiles
                if owner == r:
                    if flush_before_wait and held[(r, w)] is not None:
                        o, t = held[(r, w)]
                        flags[(o, t)] = flags.get((o, t), 0) + 1
                        held[(r, w)] = None
                        progress = True
                    if flags.get((r, (tr, tc)), 0) < ws - 1:
                        break                 # begin_tile blocks
                    prev, held[(r, w)] = held[(r, w)], None
                else:
                    prev, held[(r, w)] = held[(r, w)], (owner, (tr, tc))
                if prev is not None:          # the previous tile's hook runs after this tile's epilogue
                    o, t = prev
                    flags[(o, t)] = flags.get((o, t), 0) + 1
                pos[(r, w)] = i + 1
                progress = True
    return sum(1 for k in seqs if pos[k] < len(seqs[k]))


def simulate_pull(M, N, ws, ctas, pair):
    """Pull and scatter share this protocol. Returns (work items whose tile never got all ws
    signals, work items served by no CTA or by more than one). Also checks that every CTA meets its
    items in the order their tiles are computed (no item waits behind a later tile's)."""
    plans = [_plan(M, N, ws, r, 1, ctas, pair) for r in range(ws)]
    orders = [_order(pl) for pl in plans]
    assert all(o == orders[0] for o in orders)            # every rank walks the same order
    is_pair = bool(plans[0]["pair"])
    rows_per_tile = 256 if is_pair else 128
    slab_tiles = (M // ws) // rows_per_tile
    halves = 2 if is_pair else 1
    num_ctas = plans[0]["workers"] * halves
    SUBS = 128 // plans[0]["sub_rows"]                     # work items per 128-row tile
    assert plans[0]["sub_rows"] in (16, 32, 64, 128) and plans[0]["sub_rows"] * min(ws, 8) >= 128
    per_tile = halves * SUBS
    flags = {}
    for r in range(ws):                                   # epilogues never wait: all signals get sent
        for (tr, tc) in orders[r]:
            for h in range(halves):
                key = (tr // slab_tiles, (tr * halves + h, tc))
                flags[key] = flags.get(key, 0) + 1
    starved = wrong = 0
    order_pos = {t: i for i, t in enumerate(orders[0])}
    for r in range(ws):
        served = {}
        last_pos = {}
        tiles_r, tiles_c, group_r = plans[r]["tiles_r"], plans[r]["tiles_c"], plans[r]["group_r"]
        total_items = slab_tiles * tiles_c * per_tile
        for me in range(num_ctas):                        # the reducer warps' item -> tile arithmetic, restated
            first, gend = 0, min(group_r, tiles_r)
            v0 = r % ws
            n_g = (gend - 1 - v0) // ws + 1 if v0 < gend else 0
            o_base = 0
            for item_id in range(me, total_items, num_ctas):
                o, k = item_id // per_tile, item_id % per_tile
                while o >= o_base + n_g * tiles_c:
                    o_base += n_g * tiles_c
                    first += group_r
                    gend = min(first + group_r, tiles_r)
                    v0 = first + (r - first % ws + ws) % ws
                    n_g = (gend - 1 - v0) // ws + 1 if v0 < gend else 0
                idx = o - o_base
                tc = idx // n_g
                tr = r * slab_tiles + v0 // ws + (idx - tc * n_g)
                item = (tr * halves + k // SUBS, tc, k % SUBS)
                served[item] = served.get(item, 0) + 1
                if flags.get((r, item[:2]), 0) != ws:
                    starved += 1
                pos = order_pos[(item[0] // halves, item[1])]
                assert pos >= last_pos.get(me, -1), "items must follow the tile order"
                last_pos[me] = pos
        own_tiles = [t for t in orders[r] if t[0] // slab_tiles == r]
        expect = {(tr * halves + h, tc, j) for (tr, tc) in own_tiles for h in range(halves) for j in range(SUBS)}
        wrong += len(expect.symmetric_difference(served.keys())) + sum(1 for v in served.values() if v != 1)
    return starved, wrong


CASES = [(ws, M, N, ctas, pair)
         for ws in (2, 4, 8)
         for M in (256 * ws, 1024, 2048, 8192)
         for N in (1024, 8192)
         for (ctas, pair) in ((4, True), (12, True), (148, True), (148, False))
         if M % ws == 0 and (M // ws) % 128 == 0]


@pytest.mark.parametrize("ws,M,N,ctas,pair", CASES)
def test_push_never_blocks_while_holding_a_signal(ws, M, N, ctas, pair):
    assert simulate_push(M, N, ws, ctas, pair, flush_before_wait=True) == 0


@pytest.mark.parametrize("ws", [4, 8])
def test_model_finds_the_cycle_when_signals_are_held_across_a_wait(ws):
    # Without the flush, M = 2048, N = 8192 on 74 CTA pairs closes a wait-for cycle across ranks at
    # 4 and 8 ranks (every own tile needs a signal some peer holds back behind its own wait).
    assert simulate_push(2048, 8192, ws, 148, True, flush_before_wait=False) > 0
    assert simulate_push(2048, 8192, 2, 148, True, flush_before_wait=False) == 0


@pytest.mark.parametrize("ws,M,N,ctas,pair", CASES)
def test_pull_every_work_item_is_served_exactly_once(ws, M, N, ctas, pair):
    assert simulate_pull(M, N, ws, ctas, pair) == (0, 0)


@pytest.mark.parametrize("ws", [2, 4, 8])
def test_pull_order_interleaves_the_owners(ws):
    pl = _plan(8192, 8192, ws, 0, 1, 148, True)
    order = _order(pl)
    slab_tiles = (8192 // ws) // 256
    owners = [tr // slab_tiles for tr, _ in order]
    assert sorted(order) == [(r, c) for r in range(pl["tiles_r"]) for c in range(pl["tiles_c"])]
    # within any window of one wave (74 pair tiles) every owner gets its share, give or take a group
    W = pl["workers"]
    for start in range(0, len(order) - W, W):
        counts = [owners[start:start + W].count(o) for o in range(ws)]
        assert max(counts) - min(counts) <= pl["group_r"], (start, counts)
