"""The residency policy on the CPU (host-only mode: "device" buffers are numpy arrays, copies are
memcpy): the slab rebuild and the tables of src/core/layer.cpp:21-109, the arena's LRU rules with
the cases of the reference's own test (tests/test_expert_pump.cpp:56-135: reuse, LRU eviction, stale
residency, clear, fallback, churn) plus the rule that test could not reach on a CPU build - a slot
whose copy is in flight is never stolen - and the decode table of src/core/session.cpp:3569-3627."""
import numpy as np
import pytest

from sager_b200 import lib
from sager_b200.residency import Residency

H, F = 256, 256
L, E = 2, 8


def make(slab, arena):
    r = Residency(L, E, H, F, slab, arena)
    eb = r.expert_bytes
    rng = np.random.default_rng(3)
    pool = rng.integers(0, 256, size=L * E * eb, dtype=np.uint8)
    slab_mem = np.zeros(max(1, slab) * eb, dtype=np.uint8)
    arena_mem = np.zeros(max(1, arena) * eb, dtype=np.uint8)
    table = np.zeros(3 * L * E, dtype=np.uint64)
    r.bind(pool, slab_mem, arena_mem, table, host_only=True)
    return r, pool, slab_mem, arena_mem, table, eb


def test_rebuild_fills_the_slab_in_layer_expert_order_and_builds_both_tables():
    r, pool, slab, arena, table, eb = make(slab=5, arena=2)
    wanted = [(0, 1), (0, 6), (1, 0), (1, 3), (1, 7), (0, 3)]       # six wanted, the slab holds five
    for l, e in wanted:
        r.set_resident(l, e)
    assert r.rebuild() == 5
    order = sorted(wanted)[:5]                                      # (layer, expert) ascending; (1, 7) does not fit
    gu = eb // 3
    hot = r.host_table(1)
    for slot, (l, e) in enumerate(order):
        src = pool[(l * E + e) * eb:(l * E + e + 1) * eb]
        assert np.array_equal(slab[slot * eb:(slot + 1) * eb], src)
        base = slab.ctypes.data + slot * eb
        assert hot[l, :, e].tolist() == [base, base + gu, base + 2 * gu]
        assert r.where(l, e) == 1
    assert r.where(1, 7) == 0 and hot[1, :, 7].tolist() == [0, 0, 0]
    # one more expert through the arena, then the decode table: [3][L][E], slab first, arena second, null = absent
    slot = r.submit(1, 7, step=1)
    assert slot >= 0 and r.where(1, 7) == 2
    assert np.array_equal(arena[slot * eb:(slot + 1) * eb], pool[(1 * E + 7) * eb:(1 * E + 8) * eb])
    absent = r.build_decode_table()
    assert absent == L * E - 6 and r.absent(0) == E - 3 and r.absent(1) == E - 3
    t = table.reshape(3, L, E)
    assert np.array_equal(t, r.host_table(0))
    for l in range(L):
        for e in range(E):
            if (l, e) in order:
                assert t[:, l, e].tolist() == hot[l, :, e].tolist()
            elif (l, e) == (1, 7):
                base = arena.ctypes.data + slot * eb
                assert t[:, l, e].tolist() == [base, base + gu, base + 2 * gu]
            else:
                assert t[:, l, e].tolist() == [0, 0, 0]
    assert r.submit(0, 1, step=2) == -2                             # in the slab: no arena slot needed
    r.close()


def test_arena_reuse_lru_eviction_clear_fallback_and_churn():
    r, *_ = make(slab=0, arena=4)
    s1 = r.submit(0, 3, 1)
    assert s1 >= 0 and r.where(0, 3) == 2
    assert r.submit(0, 3, 2) == s1                                   # reuse: same slot, no new copy
    assert (r.stat(2), r.stat(3), r.stat(1)) == (1, 1, 1)
    r.close()

    r, *_ = make(slab=0, arena=2)
    a, b = r.submit(0, 0, 1), r.submit(0, 1, 2)
    assert a >= 0 and b >= 0 and a != b and r.where(1, 0) == 0
    assert r.submit(0, 1, 3) == b                                    # touch the newer one
    c = r.submit(1, 0, 4)                                            # full: evicts the least recently used
    assert c == a and r.where(0, 0) == 0 and r.where(0, 1) == 2 and r.where(1, 0) == 2
    assert r.stat(4) == 1 and r.submit(1, 0, 5) == c
    r.clear_arena()
    assert r.stat(1) == 0 and r.where(0, 1) == 0 and r.submit(0, 5, 6) >= 0
    assert r.stat(2) == 4                                            # lifetime counter survives the clear
    r.close()

    r, *_ = make(slab=0, arena=0)
    assert r.submit(0, 0, 1) == -1 and r.stat(5) == 1 and r.where(0, 0) == 0     # no arena: fallback
    r.close()

    r, *_ = make(slab=0, arena=4)
    slots = set()
    for step in range(1, 17):
        s = r.submit(step % L, (step * 3) % E, step)
        assert s >= 0
        slots.add(s)
    assert len(slots) <= 4 and r.stat(4) + r.stat(5) >= 8
    r.close()


def test_a_slot_whose_copy_is_in_flight_is_never_stolen():
    r, *_ = make(slab=0, arena=2)
    a, b = r.submit(0, 0, 1), r.submit(0, 1, 2)
    fn = lib().raw("sgr_residency_test_set_inflight")
    assert fn(r._h, a, 1) == 0                                       # the older slot is still being filled
    c = r.submit(1, 2, 3)
    assert c == b and r.where(0, 0) == 2 and r.where(0, 1) == 0      # the newer, completed slot went instead
    assert fn(r._h, b, 1) == 0
    assert r.submit(1, 3, 4) == -1 and r.stat(5) == 1                # both in flight: the caller falls back
    assert fn(r._h, a, 0) == 0
    assert r.submit(1, 3, 5) == a                                    # completed: may be reused now
    r.close()


def test_everything_resident_is_the_plain_case():
    r, pool, slab, arena, table, eb = make(slab=L * E, arena=0)
    for l in range(L):
        for e in range(E):
            r.set_resident(l, e)
    assert r.rebuild() == L * E
    assert r.build_decode_table() == 0 and all(r.absent(l) == 0 for l in range(L))
    assert np.array_equal(slab[:L * E * eb], pool)                   # (layer, expert) order = pool order
    assert np.all(table != 0)
    r.close()


def test_arguments_are_checked():
    from sager_b200.capi import SagerError
    with pytest.raises(SagerError):
        Residency(0, 8, 256, 256, 1, 1)
    r, *_ = make(slab=1, arena=1)
    with pytest.raises(SagerError):
        r.set_resident(5, 0)
    assert r.submit(0, 99, 1) == -1
    r.close()
