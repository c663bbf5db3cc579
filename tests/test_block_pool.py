"""The page pool: the reference's own unit test (tests/unit/test-block-pool.cpp:1-41) restated -- chained
hashes differ, hits are verified against stored tokens, cached pages survive being freed, touching takes a
page off the free list, least recently used pages are evicted first, exhaustion and double frees raise."""
import pytest

from iian_b200.cache.block_pool import HASH_NONE, BlockPool, PoolError, hash_block


def test_chained_hashes():
    a = hash_block(HASH_NONE, [1, 2, 3, 4])
    b = hash_block(HASH_NONE, [1, 2, 3, 5])
    assert a != b and a != HASH_NONE
    assert hash_block(a, [9, 9, 9, 9]) != hash_block(b, [9, 9, 9, 9])       # the parent is part of the hash
    assert hash_block(HASH_NONE, [1, 2, 3, 4], salt=7) != a
    assert hash_block(HASH_NONE, [1, 2, 3, 4]) == a


def test_hits_are_verified_against_the_stored_tokens():
    pool = BlockPool(8, 4)
    (b,) = pool.get_new_blocks(1)
    h = hash_block(HASH_NONE, [1, 2, 3, 4])
    pool.cache_block(b, h, [1, 2, 3, 4])
    assert pool.get_cached_block(h, [1, 2, 3, 4]) == b
    assert pool.get_cached_block(h, [1, 2, 3, 9]) == -1                     # same hash, other tokens
    assert pool.get_cached_block(h + 1, [1, 2, 3, 4]) == -1
    assert BlockPool(8, 4, enable_caching=False).get_cached_block(h, [1, 2, 3, 4]) == -1


def test_cached_pages_survive_free_and_touch_takes_them_back():
    pool = BlockPool(8, 4)
    blocks = pool.get_new_blocks(3)
    hs = []
    parent = HASH_NONE
    for i, b in enumerate(blocks):
        parent = hash_block(parent, [i] * 4)
        hs.append(parent)
        pool.cache_block(b, parent, [i] * 4)
    assert pool.num_free == 5
    pool.free_blocks(list(reversed(blocks)))
    assert pool.num_free == 8 and pool.num_cached == 3
    assert pool.get_cached_block(hs[1], [1] * 4) == blocks[1]
    pool.touch(blocks[1])
    assert pool.num_free == 7 and pool.ref[blocks[1]] == 1 and blocks[1] not in pool.free_list()
    pool.touch(blocks[1])
    assert pool.ref[blocks[1]] == 2 and pool.num_free == 7
    pool.check_invariants()


def test_free_order_uncached_first_then_least_recently_used():
    pool = BlockPool(6, 2)
    a = pool.get_new_blocks(6)
    pool.cache_block(a[0], 11, [0, 0])
    pool.cache_block(a[1], 12, [1, 1])
    pool.free_blocks([a[1], a[0]])          # cached: go to the tail in this order (a[1] evicted before a[0])
    pool.free_blocks([a[2], a[3]])          # uncached: go to the head, a[2] first
    assert pool.free_list() == [a[2], a[3], a[1], a[0]]
    got = pool.get_new_blocks(3)
    assert got == [a[2], a[3], a[1]] and pool.evictions == 1
    assert pool.get_cached_block(12, [1, 1]) == -1 and pool.get_cached_block(11, [0, 0]) == a[0]


def test_exhaustion_and_double_free_raise():
    pool = BlockPool(4, 2)
    blocks = pool.get_new_blocks(4)
    with pytest.raises(PoolError, match="out of blocks"):
        pool.get_new_blocks(1)
    pool.free_blocks(blocks[:2])
    with pytest.raises(PoolError, match="double free"):
        pool.free_blocks(blocks[:1])
    pool.check_invariants()


def test_reset_prefix_cache_only_when_idle():
    pool = BlockPool(4, 2)
    (b,) = pool.get_new_blocks(1)
    pool.cache_block(b, 5, [1, 2])
    assert not pool.reset_prefix_cache()
    pool.free_blocks([b])
    assert pool.reset_prefix_cache() and pool.num_cached == 0 and pool.get_cached_block(5, [1, 2]) == -1
