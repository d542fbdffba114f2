"""Host-side page bookkeeping of the paged latent cache (blok_kv_pages_*): runs without a GPU.

The reference's KvCache (src/kimi_exec.cu:192-238) is one contiguous region whose only rule is the capacity check at
:205; the rules tested here are the ones pages add: no page in two sequences unless forked, a full pool refuses
without side effects, released pages come back.
"""
import numpy as np
import pytest

from blok_b200 import lib


def _held(p):
    """{slot: [pages]} from the table and the reserved row counts."""
    t = p.table()
    return {s: list(t[s, :p.rows(s) // p.page_rows]) for s in range(p.slots)}


def test_reserve_grows_by_whole_pages_and_never_shares():
    p = lib.KvPages(n_pages=10, page_rows=64, slots=3, table_stride=4)
    assert p.free == 10 and p.rows(0) == 0
    p.reserve(0, 1)
    assert p.rows(0) == 64 and p.free == 9
    p.reserve(0, 64)          # still one page
    assert p.rows(0) == 64 and p.free == 9
    p.reserve(0, 65)
    p.reserve(1, 200)         # 4 pages
    assert p.rows(0) == 128 and p.rows(1) == 256 and p.free == 4
    p.reserve(0, 10)          # a reservation never shrinks
    assert p.rows(0) == 128
    held = _held(p)
    pages = held[0] + held[1]
    assert len(set(pages)) == len(pages) == 6 and all(0 <= x < 10 for x in pages)
    first = list(held[0])
    p.reserve(0, 256)         # growing keeps the pages already held, in place
    assert _held(p)[0][:2] == first
    p.close()


def test_limits_are_refused_without_side_effects():
    p = lib.KvPages(n_pages=3, page_rows=32, slots=2, table_stride=4)
    p.reserve(0, 64)
    before = (p.table().copy(), p.free, p.rows(1))
    with pytest.raises(lib.BlokError) as e:
        p.reserve(1, 65)      # needs 3 pages, 1 free
    assert e.value.code == -6
    with pytest.raises(lib.BlokError) as e:
        p.reserve(1, 4 * 32 + 1)   # more than a slot's table row holds
    assert e.value.code == -2
    with pytest.raises(lib.BlokError):
        p.reserve(2, 1)       # no such slot
    with pytest.raises(lib.BlokError):
        p.reserve(0, -1)
    assert np.array_equal(p.table(), before[0]) and p.free == before[1] and p.rows(1) == before[2]
    for bad in ((0, 64, 1, 4), (4, 48, 1, 4), (4, 0, 1, 4), (4, 64, 0, 4), (4, 64, 1, 0)):
        with pytest.raises(lib.BlokError):
            lib.KvPages(*bad)
    p.close()


def test_release_returns_pages_and_they_are_reused():
    p = lib.KvPages(n_pages=4, page_rows=32, slots=4, table_stride=4)
    p.reserve(0, 64)
    p.reserve(1, 64)
    assert p.free == 0
    mine = set(_held(p)[0])
    p.release(0)
    assert p.free == 2 and p.rows(0) == 0 and not p.table()[0].any()
    p.reserve(2, 64)
    assert set(_held(p)[2]) == mine
    p.release(3)              # releasing an empty slot is a no-op
    assert p.free == 0
    p.close()


def test_fork_shares_whole_prefix_pages_until_the_last_holder_leaves():
    p = lib.KvPages(n_pages=6, page_rows=32, slots=3, table_stride=4)
    p.reserve(0, 96)
    base = _held(p)[0]
    with pytest.raises(lib.BlokError):
        p.fork(0, 1, 40)      # not a whole number of pages
    with pytest.raises(lib.BlokError):
        p.fork(0, 1, 128)     # more than the source holds
    with pytest.raises(lib.BlokError):
        p.fork(0, 0, 32)
    p.fork(0, 1, 64)
    assert _held(p)[1] == base[:2] and p.free == 3
    p.reserve(1, 96)          # the continuation gets a page of its own
    own = _held(p)[1][2]
    assert own not in base and p.free == 2
    with pytest.raises(lib.BlokError):
        p.fork(0, 1, 32)      # the destination must be empty
    p.release(0)              # the shared pages stay with slot 1; only the unshared third page returns
    assert p.free == 3 and _held(p)[1] == base[:2] + [own]
    p.release(1)
    assert p.free == 6
    p.close()


def test_random_sequence_lifecycle_conserves_pages():
    rng = np.random.default_rng(0)
    n_pages, rows, slots, stride = 40, 32, 8, 12
    p = lib.KvPages(n_pages, rows, slots, stride)
    length = [0] * slots
    for _ in range(2000):
        s = int(rng.integers(slots))
        if rng.random() < 0.15:
            p.release(s)
            length[s] = 0
        else:
            want = min(length[s] + int(rng.integers(1, 70)), stride * rows)
            try:
                p.reserve(s, want)
                length[s] = want
            except lib.BlokError as e:
                assert e.code == -6
        held = _held(p)
        flat = [x for v in held.values() for x in v]
        assert len(set(flat)) == len(flat)                      # no page in two sequences
        assert len(flat) + p.free == n_pages                    # none lost
        assert all(p.rows(i) >= length[i] for i in range(slots))
        assert all(p.rows(i) - length[i] < rows or length[i] == 0 and p.rows(i) == 0 for i in range(slots))
    p.close()
