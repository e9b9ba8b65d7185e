"""The balanced last wave of the tensor-core GEMM, checked on the CPU through the library's own arithmetic
(pg_b200_debug_tail_schedule runs the very function the kernel's roles call): with T tiles on S resident CTA pairs
and T % S != 0, the K ranges of the T % S tail tiles are dealt out to all S pairs so that

  * every tail tile is covered exactly once, by one whole part or by a first slice [0, s) and a second slice [s, KB);
  * no tile has more than two slices (two terms per element, added in one order: deterministic);
  * the pairs of a group of k tiles and k + 1 pairs each get k / (k + 1) of a tile (k differs by at most one
    between groups);
  * a pair that holds a first and a second slice is given the first slice first (the order that keeps the
    second slice's wait for the first short).
"""
import ctypes

import pytest

from picograd_b200._lib import lib


def schedule(tiles, slots, kb):
    parts = {}
    used = full = None
    for c in range(slots):
        for j in (0, 1):
            out = (ctypes.c_uint * 6)()
            assert lib.pg_b200_debug_tail_schedule(tiles, slots, kb, c, j, out) == 0
            used, full = out[0], out[1]
            if out[4]:
                parts[(c, j)] = (out[2], out[3], out[4], out[5])
    return used, full, parts


@pytest.mark.parametrize("tiles,slots,kb", [(128, 74, 128), (256, 74, 128), (128, 74, 32), (48, 74, 128), (96, 74, 18),
                                            (75, 74, 64), (147, 74, 64), (10, 74, 256), (73, 74, 128), (200, 148, 40)])
def test_tail_tiles_are_covered_once_and_evenly(tiles, slots, kb):
    used, full, parts = schedule(tiles, slots, kb)
    if not used:
        assert not parts
        return
    assert full == tiles // slots
    rem = tiles % slots
    cover = {t: [] for t in range(rem)}
    load = [0] * slots
    for (c, j), (tile, b, n, role) in parts.items():
        assert tile < rem and role in (1, 2)
        cover[tile].append((b, n, role, c, j))
        load[c] += n
    for t, segs in cover.items():
        segs.sort()
        assert len(segs) == 2, (t, segs)
        (b0, n0, r0, c0, _), (b1, n1, r1, c1, _) = segs
        assert b0 == 0 and r0 == 1 and b1 == n0 and r1 == 2 and b1 + n1 == kb and n0 >= 1 and n1 >= 1
        assert c0 != c1
    for c in range(slots):
        mine = sorted((j, parts[(c, j)][3]) for j in (0, 1) if (c, j) in parts)
        if len(mine) == 2:
            assert [r for _, r in mine] == [1, 2]          # first slice first
    # groups of k tiles on k + 1 pairs: every pair of a group multiplies k / (k + 1) of a tile; k is q or q + 1
    groups = slots - rem
    q, r = divmod(rem, groups)
    kmax = q + (1 if r else 0)
    assert max(load) <= kb * kmax / (kmax + 1) + 1
    busy = [x for x in load if x]
    if q >= 1:
        assert len(busy) == slots and min(busy) >= kb * q / (q + 1) - 1
    else:
        assert len(busy) == 2 * rem and min(busy) >= kb // 2 - 1


def test_many_waves_keep_the_plain_schedule():
    # 1024 tiles of 8192^3 on 74 pairs: the last wave is 62/74 full and one of fourteen: not worth a second slice
    used, _, parts = schedule(1024, 74, 128)
    assert not used and not parts
    # full waves: nothing to balance
    assert not schedule(148, 74, 128)[0]
    # short K: a slice would be shorter than four blocks
    assert not schedule(128, 74, 8)[0]
