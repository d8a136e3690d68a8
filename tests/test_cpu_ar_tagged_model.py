"""Host model of the wait-for order of the tagged exchanges of the decode GEMM -> all-reduce
(csrc/include/kraken/gemm_hooks.cuh: helper_role, two_shot_tagged).

Every CTA (the same grid on every rank) walks its work items t = bid, bid + nb, ... twice: first it
computes each item and pushes its partial sums (never waiting), then it walks them again and either
sums and publishes (the tile's owner, tile % ws) or waits for the owner's published share of that
item (the other ranks). The model runs the second walk to a fixed point, with the partials of a
CTA counted as available only once that CTA has finished its first walk, and CTAs scheduled in an
adversarial order; a CTA that can never advance is a deadlock.

It also restates the slot / offset arithmetic of the packed partial arrays and checks that no two
writers share a pair and that every pair a reader polls has exactly one writer.
"""
import itertools

import pytest


def simulate(ws, tiles, ks, nb, order):
    """Returns the number of (rank, cta) pairs that never finish. `order` permutes the schedule."""
    total = tiles * ks
    ctas = [(r, b) for r in range(ws) for b in range(nb)]
    seq = {c: list(range(c[1], total, nb)) for c in ctas}
    pushed = set()          # (rank, cta) whose first walk is over: all its partials are out
    pos = {c: 0 for c in ctas}
    published = set()       # (owner rank, item)
    sched = [ctas[i] for i in order(len(ctas))]
    progress = True
    while progress:
        progress = False
        for c in sched:
            if c not in pushed:
                pushed.add(c)              # the first walk waits for nothing
                progress = True
                continue
            r, b = c
            while pos[c] < len(seq[c]):
                t = seq[c][pos[c]]
                tile = t % tiles
                owner = tile % ws
                if owner == r:
                    # needs the partials of this tile from every rank and split: item (split', tile) belongs to
                    # CTA (split' * tiles + tile) % nb on each rank
                    need = [(rr, (s * tiles + tile) % nb) for rr in range(ws) for s in range(ks)]
                    if not all(n in pushed for n in need):
                        break
                    published.add((r, t))
                elif (owner, t) not in published:
                    break
                pos[c] += 1
                progress = True
    return sum(1 for c in ctas if pos[c] < len(seq[c]))


ORDERS = {
    "forward": lambda n: list(range(n)),
    "backward": lambda n: list(range(n - 1, -1, -1)),
    "interleaved": lambda n: list(range(0, n, 2)) + list(range(1, n, 2)),
}


@pytest.mark.parametrize("ws", [2, 3, 4, 8])
@pytest.mark.parametrize("order", sorted(ORDERS))
def test_tagged_two_shot_never_deadlocks(ws, order):
    for tiles, ks in itertools.product((1, 2, 5, 8, 16, 64), (1, 2, 4)):
        total = tiles * ks
        for nb in sorted({1, 2, 3, max(1, total // 3), max(1, total - 1), total}):
            assert simulate(ws, tiles, ks, nb, ORDERS[order]) == 0, (ws, tiles, ks, nb)


def test_model_detects_a_wait_before_the_own_pushes_are_out():
    # If a CTA waited for a peer's published result BEFORE pushing its own later items, two ranks
    # could wait for each other. The model shows it when the first walk is not allowed to complete.
    ws, tiles, ks, nb = 2, 2, 1, 1
    total = tiles * ks
    pos = {r: 0 for r in range(ws)}
    pushed_items = {r: set() for r in range(ws)}
    published = set()
    progress = True
    while progress:
        progress = False
        for r in range(ws):
            while pos[r] < total:
                t = pos[r]
                pushed_items[r].add(t)                       # push item t, then try to finish it at once
                owner = t % ws
                if owner == r:
                    if not all(t in pushed_items[rr] for rr in range(ws)):
                        break
                    published.add((r, t))
                elif (owner, t) not in published:
                    break
                pos[r] += 1
                progress = True
    assert any(pos[r] < total for r in range(ws))            # rank 0 waits at item 0 for rank 1, which waits at item 0 too


@pytest.mark.parametrize("ws,tiles,ks,bn,rows", [(2, 8, 1, 16, 1), (4, 16, 2, 16, 5), (8, 64, 1, 16, 16), (8, 128, 1, 32, 64), (3, 7, 2, 64, 40)])
def test_packed_partial_arrays_have_one_writer_per_pair(ws, tiles, ks, bn, rows):
    """Restates the addressing of the tagged two-shot: slot = rank * ks + split; inside a slot the
    tiles of one owner are packed in order (tile // ws), bn x 128 pairs each."""
    per_slot = -(-tiles // ws) * bn * 128
    region_pairs = ws * ks * per_slot
    for owner in range(ws):
        written = {}
        for src in range(ws):
            for split in range(ks):
                slot = src * ks + split
                for tile in range(owner, tiles, ws):
                    base = slot * per_slot + (tile // ws) * bn * 128
                    for lr in sorted({0, min(rows, bn) - 1}):
                        for lc in (0, 127):
                            off = base + lr * 128 + lc
                            assert 0 <= off < region_pairs
                            assert off not in written, "two writers for one pair"
                            written[off] = (src, split, tile)
        # the owner reads, for each of its tiles, the same pair of every slot
        for tile in range(owner, tiles, ws):
            for slot in range(ws * ks):
                off = slot * per_slot + (tile // ws) * bn * 128
                assert written.get(off) == (slot // ks, slot % ks, tile)
