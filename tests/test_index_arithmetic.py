"""CPU checks of the fused kernels' index arithmetic, run on the host build of the very
functions the kernels use (tile decoding, sender tables).  They cover what a single GPU
cannot: the cross-rank row layout for worlds of 2, 4 and 8."""
import ctypes as C
import random

import pytest


def _lib():
    from iris_testing_b200 import _native
    try:
        return _native.lib()
    except Exception as exc:
        pytest.skip(f"native library unavailable: {exc}")


def tile_order(lib, rows, TN, gm, tile_rows):
    G = len(rows)
    total = sum((r + tile_rows - 1) // tile_rows for r in rows) * TN
    out = (C.c_int * (3 * max(total, 1)))()
    arr = (C.c_int * G)(*rows)
    n = lib.b200_debug_tile_order(arr, G, TN, gm, tile_rows, out, max(total, 1))
    assert n == total, n
    return [(out[3 * i], out[3 * i + 1], out[3 * i + 2]) for i in range(total)]


@pytest.mark.parametrize("tile_rows", [128, 256])
def test_every_tile_is_scheduled_exactly_once(tile_rows):
    lib = _lib()
    rng = random.Random(tile_rows)
    for _ in range(60):
        G = rng.randint(1, 40)
        rows = [rng.choice([0, 0, 1, 5, 127, 128, 129, 255, 256, 257, 1000, rng.randint(0, 5000)]) for _ in range(G)]
        TN, gm = rng.randint(1, 20), rng.randint(1, 16)
        tiles = tile_order(lib, rows, TN, gm, tile_rows)
        expected = {(g, m, n) for g, r in enumerate(rows) for m in range((r + tile_rows - 1) // tile_rows)
                    for n in range(TN)}
        assert len(tiles) == len(expected) and set(tiles) == expected
        # groups are visited in order, and inside a chunk the M index runs fastest
        assert [t[0] for t in tiles] == sorted(t[0] for t in tiles)
        for (g0, m0, n0), (g1, m1, n1) in zip(tiles, tiles[1:]):
            if g0 == g1 and n0 == n1 and m1 != m0 + 1:
                assert m1 < m0 or n1 != n0     # a new chunk or a new N column starts


def test_chunks_are_evened_out():
    lib = _lib()
    tiles = tile_order(lib, [16 * 256], 3, 12, 256)          # 16 M-tiles, target 12 -> two chunks of 8
    first_column = [m for (g, m, n) in tiles if n == 0]
    assert first_column[:8] == list(range(8)) and tiles[8][2] == 1


def test_even_rounds_tile_walk_covers_every_tile_in_the_minimum_number_of_rounds():
    """The persistent kernels' tile walk: every tile has exactly one owner, nobody takes more than
    ceil(tiles / schedulers) tiles (the number of rounds is not increased), and the tiles are
    spread over as few schedulers as that allows, each with a full share."""
    lib = _lib()
    rng = random.Random(5)
    cases = [(0, 1), (1, 1), (1, 148), (75, 74), (896, 148), (896, 74), (128, 148), (14336, 74), (149, 148)]
    cases += [(rng.randint(0, 3000), rng.randint(1, 148)) for _ in range(200)]
    for total, sched in cases:
        owner = (C.c_int * max(total, 1))()
        assert lib.b200_debug_tile_walk(total, sched, owner) == 0, (total, sched)
        own = list(owner)[:total]
        assert all(0 <= o < sched for o in own), (total, sched)
        if total == 0:
            continue
        rounds = -(-total // sched)
        per = {}
        for o in own:
            per[o] = per.get(o, 0) + 1
        assert max(per.values()) == rounds, (total, sched)
        assert len(per) == -(-total // rounds) and min(per.values()) >= rounds - 1, (total, sched, len(per))
    # the shape that motivated it: 896 tiles on 148 CTAs are 7 rounds either way; 128 CTAs take 7 each
    owner = (C.c_int * 896)()
    lib.b200_debug_tile_walk(896, 148, owner)
    assert max(owner) == 127


def dispatch_tables(lib, counts, W, EL, rank, cap):
    ET = W * EL
    flat = [counts[s][d][e] for s in range(W) for d in range(W) for e in range(EL)]
    arr = (C.c_int * len(flat))(*flat)
    g_rows = (C.c_int * EL)()
    tables = (C.c_int * (7 * ET))()
    ok = lib.b200_debug_dispatch_tables(arr, W, EL, rank, cap, g_rows, tables)
    t = [[tables[k * ET + b] for b in range(ET)] for k in range(7)]
    return ok, list(g_rows), dict(count=t[0], send_start=t[1], dst_row=t[2], rel0=t[3], mtile0=t[4],
                                  dst_rank=t[5], units=t[6])


@pytest.mark.parametrize("W,EL", [(1, 8), (2, 4), (4, 2), (8, 1), (8, 16), (4, 32), (1, 128)])
def test_cross_rank_row_layout_is_a_partition(W, EL):
    """For every destination rank and expert, the row ranges that the sources compute for
    themselves tile that expert's block exactly, in the order self, self-1, self-2, ...;
    send offsets follow the packed (destination, expert) order of the sender."""
    lib = _lib()
    rng = random.Random(W * 1000 + EL)
    for trial in range(6):
        counts = [[[rng.choice([0, 0, 1, 31, 32, 33, 127, 128, 300, rng.randint(0, 700)]) for _ in range(EL)]
                   for _ in range(W)] for _ in range(W)]
        cap = 1 << 24
        per_rank = [dispatch_tables(lib, counts, W, EL, r, cap) for r in range(W)]
        for dst in range(W):
            rows_e = [sum(counts[s][dst][e] for s in range(W)) for e in range(EL)]
            assert per_rank[dst][1] == rows_e                      # receiver's view of its groups
            group_start = [sum(rows_e[:e]) for e in range(EL)]
            mtile0 = [sum((r + 127) // 128 for r in rows_e[:e]) for e in range(EL)]
            for e in range(EL):
                expect_row = group_start[e]
                for q in range(W):                                 # arrival order of the sources
                    src = (dst - q) % W
                    ok, _, t = per_rank[src]
                    assert ok == 1
                    bi = e * W + (dst - src) % W                   # src's bucket index for (dst, e)
                    assert t["dst_rank"][bi] == dst and t["count"][bi] == counts[src][dst][e]
                    assert t["dst_row"][bi] == expect_row and t["rel0"][bi] == expect_row - group_start[e]
                    assert t["mtile0"][bi] == mtile0[e]
                    n = counts[src][dst][e]
                    rel0 = t["rel0"][bi]
                    units = ((rel0 + n - 1) // 32 - rel0 // 32 + 1) if n else 0
                    assert t["units"][bi] == units
                    expect_row += n
                assert expect_row == group_start[e] + rows_e[e]
        for src in range(W):                                        # packed send order of the sender
            t = per_rank[src][2]
            flat = [counts[src][d][e] for d in range(W) for e in range(EL)]
            for bi in range(W * EL):
                e, r = divmod(bi, W)
                ge = ((src + r) % W) * EL + e
                assert t["send_start"][bi] == sum(flat[:ge])


def test_receive_capacity_overflow_is_flagged():
    lib = _lib()
    W, EL = 2, 1
    counts = [[[100], [50]], [[200], [60]]]          # counts[src][dst][e]
    ok, rows, _ = dispatch_tables(lib, counts, W, EL, 0, 299)      # rank 0 receives 300 rows
    assert rows == [300]
    assert dispatch_tables(lib, counts, W, EL, 1, 299)[0] == 0     # rank 1's rows for rank 0 would not fit
    assert dispatch_tables(lib, counts, W, EL, 1, 300)[0] == 1
