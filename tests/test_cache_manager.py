"""The cache manager: block tables per request and group, all-or-nothing allocation, windows that give
pages back, prefix reuse, state slots -- and that under random orders of requests no page is lost, held
twice or freed twice."""
import random

import pytest

from iian_b200.cache.block_pool import PoolError
from iian_b200.cache.manager import CacheManager, PageGroup, StateSlots


def manager(blocks=16, bs=4, window=None, caching=True, slots=4, window_blocks=None):
    groups = [PageGroup("full", (0, 1), None, blocks)]
    if window:
        groups.append(PageGroup("win", (2,), window, window_blocks or blocks))
    return CacheManager(groups, bs, caching, slots)


def held(rc, g=0):
    return [p for p in rc.tables[g] if p >= 0]


def test_allocation_grows_the_table_and_is_all_or_nothing():
    m = manager(blocks=4, bs=4)
    a, b = m.new_request(), m.new_request()
    assert m.allocate(a, 0, 5) and len(a.tables[0]) == 2
    assert m.allocate(a, 5, 1) and len(a.tables[0]) == 2          # still fits the second page
    assert m.allocate(a, 6, 3) and len(a.tables[0]) == 3
    assert not m.allocate(b, 0, 8)                                 # needs 2, only 1 free
    assert b.tables[0] == [] and m.num_free() == 1                 # nothing was taken
    assert m.allocate(b, 0, 4)
    assert m.slot_of(a, 0, 5) == a.tables[0][1] * 4 + 1
    m.free(a)
    m.free(b)
    assert m.num_free() == 4
    m.check_invariants()


def test_every_group_or_none():
    m = manager(blocks=8, bs=4, window=6, window_blocks=2)
    a = m.new_request()
    assert not m.allocate(a, 0, 12)                # the windowed group cannot hold 3 pages at once
    assert a.tables == [[], []] and m.num_free(0) == 8 and m.num_free(1) == 2
    assert m.allocate(a, 0, 8)


def test_window_gives_pages_back_while_the_request_runs():
    m = manager(blocks=16, bs=4, window=6)
    a = m.new_request()
    pos = 0
    for n in (5, 3, 1, 1, 1, 1, 7, 1):
        assert m.allocate(a, pos, n)
        pos += n
        first = m.first_needed_block(1, pos)
        # after the step the next query is at `pos` and sees keys > pos - 6
        m.release_passed(a, pos)
        assert all(p == -1 for p in a.tables[1][:first]) and all(p >= 0 for p in a.tables[1][first:])
        assert all(p >= 0 for p in a.tables[0])                    # the full group keeps everything
    assert m.first_needed_block(1, 20) == (20 - 6 + 1) // 4
    with pytest.raises(PoolError, match="given back"):
        m.slot_of(a, 1, 0)
    m.free(a)
    assert m.num_free(0) == 16 and m.num_free(1) == 16
    m.check_invariants()


def test_prefix_reuse_full_pages_only_and_never_the_last_token():
    m = manager(blocks=16, bs=4)
    toks = list(range(100, 113))                   # 13 tokens: 3 full pages
    a = m.new_request()
    m.update_hashes(a, toks)
    assert len(a.hashes) == 3
    assert m.find_cached_prefix(toks, a.hashes)[0] == 0
    assert m.allocate(a, 0, 13)
    m.commit(a, toks, 13)
    b = m.new_request()
    m.update_hashes(b, toks)
    n, tables = m.find_cached_prefix(toks, b.hashes)
    assert n == 12 and tables[0] == a.tables[0][:3]
    # 12 tokens that are all cached: the last token must still be computed
    n12, t12 = m.find_cached_prefix(toks[:12], b.hashes[:3])
    assert n12 == 8 and t12[0] == a.tables[0][:2]
    assert m.allocate(b, n, 1, tables)
    assert b.tables[0][:3] == a.tables[0][:3] and m.pools[0].ref[a.tables[0][0]] == 2
    m.free(a)
    assert m.pools[0].ref[b.tables[0][0]] == 1                      # still held by b
    m.free(b)
    assert m.num_free() == 16
    # freed but cached: a third request finds them and takes them off the free list
    c = m.new_request()
    m.update_hashes(c, toks)
    n, tables = m.find_cached_prefix(toks, c.hashes)
    assert n == 12 and m.allocate(c, n, 1, tables) and m.num_free() == 12
    other = toks[:4] + [1, 2, 3, 4, 5]
    d = m.new_request()
    m.update_hashes(d, other)
    assert m.find_cached_prefix(other, d.hashes)[0] == 4            # stops at the first page that differs
    m.check_invariants()


def test_prefix_reuse_with_a_window_needs_only_the_pages_in_the_window():
    m = manager(blocks=16, bs=4, window=6)
    toks = list(range(50, 71))                     # 21 tokens: 5 full pages
    a = m.new_request()
    m.update_hashes(a, toks)
    pos = 0
    for n in (9, 8, 4):
        assert m.allocate(a, pos, n)
        pos += n
        m.commit(a, toks, pos)
    m.free(a)
    b = m.new_request()
    m.update_hashes(b, toks)
    n, tables = m.find_cached_prefix(toks, b.hashes)
    assert n == 20
    first = m.first_needed_block(1, 20)
    assert tables[1][:first] == [-1] * first and all(p >= 0 for p in tables[1][first:])
    assert all(p >= 0 for p in tables[0])
    assert m.allocate(b, n, 1, tables)
    m.free(b)
    m.check_invariants()


def test_state_slots():
    s = StateSlots(2)
    a, b = s.allot(), s.allot()
    assert {a, b} == {0, 1} and s.allot() == -1
    s.release(a)
    with pytest.raises(PoolError, match="released twice"):
        s.release(a)
    assert s.allot() == a
    m = manager(slots=1)
    r1, r2 = m.new_request(), m.new_request()
    assert m.allot_state(r1) and r1.state_fresh and not m.allot_state(r2)
    m.free(r1)
    assert r1.state_slot == -1 and m.allot_state(r2)


@pytest.mark.parametrize("seed", range(8))
@pytest.mark.parametrize("window", [None, 10])
def test_random_orders_lose_no_page(seed, window):
    """Requests arrive, grow by random portions, finish or are dropped in random order; some share
    prefixes.  After every operation each page is referenced exactly as often as tables hold it, and in
    the end every page is free again."""
    rng = random.Random(seed)
    bs = 4
    m = manager(blocks=24, bs=bs, window=window, caching=True, slots=6, window_blocks=24)
    live = []          # (cache, tokens, computed)
    prefixes = [[rng.randrange(50) for _ in range(12)] for _ in range(2)]

    def check():
        m.check_invariants()
        for g, pool in enumerate(m.pools):
            want = [0] * pool.num_blocks
            for rc, _, _ in live:
                for p in rc.tables[g]:
                    if p >= 0:
                        want[p] += 1
            assert want == pool.ref, f"group {g}: reference counts do not match the tables"

    for step in range(400):
        op = rng.random()
        if op < 0.3 and len(live) < 6:
            toks = (rng.choice(prefixes)[:] if rng.random() < 0.6 else []) + [rng.randrange(50) for _ in range(rng.randrange(1, 30))]
            rc = m.new_request()
            if not m.allot_state(rc):
                continue
            m.update_hashes(rc, toks)
            n, tables = m.find_cached_prefix(toks, rc.hashes)
            n_new = min(len(toks) - n, rng.randrange(1, 9))
            if m.allocate(rc, n, n_new, tables):
                live.append([rc, toks, n + n_new])
                m.commit(rc, toks, n + n_new)
            else:
                m.free(rc)
        elif op < 0.8 and live:
            ent = rng.choice(live)
            rc, toks, done = ent
            if done == len(toks):
                toks.append(rng.randrange(50))         # a decoded token
            n_new = min(len(toks) - done, rng.randrange(1, 7))
            if m.allocate(rc, done, n_new):
                ent[2] = done + n_new
                m.update_hashes(rc, toks)
                m.commit(rc, toks, ent[2])
            else:                                       # out of pages: drop this request (a preemption)
                m.free(rc)
                live.remove(ent)
        elif live:
            ent = rng.choice(live)
            m.free(ent[0])
            live.remove(ent)
        check()
    for rc, _, _ in live:
        m.free(rc)
    live.clear()
    check()
    assert all(p.num_free == p.num_blocks for p in m.pools)
    assert m.slots.num_free == 6
