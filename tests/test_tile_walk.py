"""The order in which the tensor-core GEMM's CTA pairs take the output tiles, checked on the CPU through the
library's own arithmetic (pg_b200_debug_walk runs the function the kernel's roles call):

  * whatever the options, every tile is taken exactly once;
  * consecutive tiles of a pair stay in one rasterisation group as long as the group lasts (same rows of A);
  * with `serpentine` the first tiles of a group are the N tiles the group before ended on;
  * with `k_serpentine` a pair's tiles alternate K upwards / downwards, so a tile begins on the K blocks the
    pair's previous tile ended on;
  * the die-aware walk gives each die one half of every group's M tiles.
"""
import ctypes
import itertools

import pytest

from picograd_b200._lib import lib


def walk(m_tiles, n_tiles, group_m, count, die_aware=0, serp=1, kserp=1, die=0, k_blocks=128):
    """[(pair, i, m, n, k_down)] for all pairs (of one die when die-aware)."""
    out = []
    for pid in range(count):
        for i in itertools.count():
            o = (ctypes.c_uint * 4)()
            assert lib.pg_b200_debug_walk(m_tiles, n_tiles, group_m, k_blocks, die_aware, serp, kserp, die, pid, count, i, o) == 0
            if not o[0]:
                break
            out.append((pid, i, o[1], o[2], o[3]))
    return out


@pytest.mark.parametrize("m_tiles,n_tiles,group_m,count", [(32, 32, 8, 74), (32, 4, 8, 74), (16, 56, 8, 74), (5, 7, 3, 4),
                                                           (33, 9, 8, 74), (1, 100, 1, 74), (64, 64, 10, 148)])
@pytest.mark.parametrize("serp,kserp", [(0, 0), (1, 0), (1, 1)])
def test_every_tile_once(m_tiles, n_tiles, group_m, count, serp, kserp):
    units = walk(m_tiles, n_tiles, group_m, count, 0, serp, kserp)
    tiles = sorted((m, n) for _, _, m, n, _ in units)
    assert tiles == [(m, n) for m in range(m_tiles) for n in range(n_tiles)]
    for pid, i, _, _, k_down in units:
        assert k_down == (i & 1 if kserp else 0)


def test_serpentine_groups_start_where_the_previous_one_ended():
    m_tiles, n_tiles, group_m, count = 32, 32, 8, 74
    order = {}
    for pid, i, m, n, _ in walk(m_tiles, n_tiles, group_m, count):
        order[pid + i * count] = (m, n)                 # position in the global walk
    seq = [order[j] for j in range(m_tiles * n_tiles)]
    per_group = group_m * n_tiles
    for g in range(1, m_tiles // group_m):
        last_n = {n for _, n in seq[g * per_group - count:g * per_group]}
        first_n = {n for _, n in seq[g * per_group:g * per_group + count]}
        assert last_n == first_n, g                     # the B panels of the wave before are the wave's own
    # within a group all tiles share the group's M tiles
    for g in range(m_tiles // group_m):
        assert {m // group_m for m, _ in seq[g * per_group:(g + 1) * per_group]} == {g}


@pytest.mark.parametrize("serp", [0, 1])
def test_die_aware_halves(serp):
    m_tiles, n_tiles, group_m, per_die = 32, 32, 8, 37
    seen = []
    for die in (0, 1):
        units = walk(m_tiles, n_tiles, group_m, per_die, 1, serp, 1, die)
        for _, _, m, _, _ in units:
            assert (m % group_m) // (group_m // 2) == die          # upper half of each group on die 0, lower on die 1
        seen += [(m, n) for _, _, m, n, _ in units]
    assert sorted(seen) == [(m, n) for m in range(m_tiles) for n in range(n_tiles)]


def test_refusals():
    o = (ctypes.c_uint * 4)()
    assert lib.pg_b200_debug_walk(0, 4, 8, 16, 0, 1, 1, 0, 0, 74, 0, o) != 0
    assert lib.pg_b200_debug_walk(32, 32, 7, 16, 1, 1, 1, 0, 0, 37, 0, o) != 0      # die-aware needs an even group
    assert lib.pg_b200_debug_walk(32, 32, 8, 16, 0, 1, 1, 0, 80, 74, 0, o) != 0     # pair beyond the count
