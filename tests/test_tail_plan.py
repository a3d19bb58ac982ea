"""The schedule of the FFMA matmul's tail wave (basalt_rt_tail_plan) against a model of what the kernels do with it.

The emitted kernel (emit_mma.cpp, sgemm_ffma) and its hand-written twin (kernels/sgemm.cu) turn {full, per, units}
into segments with the arithmetic restated in `segments_of` below; here that arithmetic is run for every unit of many
plans and checked for what the kernels rely on: every K slab of every tail tile is computed exactly once, no unit is
empty, a unit never needs more than its two workspace slots, and the units a tile's last segment sums over
(u_first .. u_last, the first one in slot 2u + 1, the others in 2u) are exactly the units that left a partial there.
"""
import ctypes as C
from collections import defaultdict

import numpy as np
import pytest

from basalt_b200 import _lib


def plan(tiles, slots, k, rounds):
    out = (C.c_uint32 * 3)()
    _lib.lib.basalt_rt_tail_plan(tiles, slots, k, rounds, out)
    return int(out[0]), int(out[1]), int(out[2])


def segments_of(unit, per, total, nkt):
    """(tail tile, first slab, slabs) of every segment of one stream unit, as the kernels walk them."""
    it0, it1 = unit * per, min(unit * per + per, total)
    while it0 < it1:
        t, k0 = divmod(it0, nkt)
        nk = min(nkt - k0, it1 - it0)
        yield t, k0, nk
        it0 += nk


def check(tiles, slots, k, rounds):
    full, per, units = plan(tiles, slots, k, rounds)
    nkt = k // 16
    if units == 0:
        assert full == tiles and per == 0
        return False
    tail = tiles - full
    total = tail * nkt
    assert tail == tiles % slots and 0 < per < nkt
    assert (units - 1) * per < total <= units * per                      # the last unit has work, none lies past the end
    assert units <= slots * max(rounds, 1)
    covered = np.zeros(total, np.int32)
    slot_owner = {}
    partials = defaultdict(list)
    for u in range(units):
        segs = list(segments_of(u, per, total, nkt))
        assert segs
        for t, k0, nk in segs:
            covered[t * nkt + k0:t * nkt + k0 + nk] += 1
            if nk != nkt:                                                # anything but a whole tile goes through the workspace
                slot = 2 * u + (1 if k0 == 0 else 0)
                assert slot not in slot_owner, (tiles, k, rounds, u)
                slot_owner[slot] = t
                partials[t].append((u, slot))
    assert (covered == 1).all()
    assert max(slot_owner) < 2 * units and max(partials) < tail          # workspace slots and tickets the launch provides
    for t, got in partials.items():
        u_first, u_last = t * nkt // per, ((t + 1) * nkt - 1) // per
        assert len(got) >= 2
        assert got == [(u, 2 * u + (1 if u == u_first else 0)) for u in range(u_first, u_last + 1)], (tiles, k, rounds, t)
    return True


@pytest.mark.parametrize("tiles,k,rounds,want", [
    (1024, 4096, 1, (888, 118, 296)),     # 4096^3: three whole waves, 136 tiles by one unit per slot
    (256, 4096, 2, (0, 111, 591)),        # a 1024-row shard under a gathering launch: two rounds
    (128, 4096, 2, (0, 56, 586)),         # a 512-row shard
    (300, 64, 1, (296, 1, 16)),           # four tail tiles of four slabs: one slab to a unit
    (300, 48, 1, (296, 1, 12)),
    (304, 16, 1, (304, 0, 0)),            # one slab per tile: nothing to cut
    (1184, 32, 1, (1184, 0, 0)),          # no tail
    (290, 4096, 1, (290, 0, 0)),          # 0.98 of a wave: not worth the partial sums
])
def test_known_plans_on_296_slots(tiles, k, rounds, want):
    assert plan(tiles, 296, k, rounds) == want
    check(tiles, 296, k, rounds)


def test_every_slab_once_over_many_shapes():
    rng = np.random.default_rng(7)
    streamed = 0
    for _ in range(1500):
        slots = int(rng.choice([296, 264, 148, 2, 1]))
        tiles = int(rng.integers(1, 4 * slots + 40))
        k = 16 * int(rng.integers(1, 513))
        rounds = int(rng.integers(0, 5))
        streamed += check(tiles, slots, k, rounds)
    assert streamed > 300


def test_degenerate_arguments_mean_no_stream_units():
    assert plan(100, 0, 4096, 1) == (100, 0, 0)
    assert plan(100, 296, 8, 1) == (100, 0, 0)
    assert plan(0, 296, 4096, 1) == (0, 0, 0)
    assert plan(295, 296, 2 ** 28, 1) == (295, 0, 0)                      # 295 x 2^24 slabs, past 2^31: left alone
