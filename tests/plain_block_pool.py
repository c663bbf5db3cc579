"""The block pool in plain Python: the model that the native pool (include/iian_b200/block_pool.h) is tested
against, operation by operation.

A pool of fixed-size cache pages with reference counts, a free list and a prefix index.

Behaviour follows the reference's ``BlockPool`` (include/iian/kv_cache.h:40-90,
src/iian/kv_cache.cpp:34-132):

* new pages come from the head of the free list; a page that still carries a prefix hash
  loses it at that moment, not when it is freed (kv_cache.cpp:93-102);
* a freed page without a hash goes to the head (used again first), one with a hash to the
  tail (kept for prefix reuse, least recently used evicted first) (kv_cache.cpp:104-116);
* a prefix hit must match the stored token ids, not just the hash (kv_cache.cpp:77-85);
* taking more pages than are free, or freeing a page twice, raises (kv_cache.cpp:94, :108).

No device memory is touched here; pages are numbers.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Tuple

HASH_NONE = 0
_MASK = (1 << 64) - 1


def _mix64(h: int) -> int:
    h &= _MASK
    h ^= h >> 33
    h = (h * 0xFF51AFD7ED558CCD) & _MASK
    h ^= h >> 33
    h = (h * 0xC4CEB9FE1A85EC53) & _MASK
    h ^= h >> 33
    return h


def hash_block(parent: int, tokens: Sequence[int], salt: int = 0) -> int:
    """Chained 64-bit hash of one full page of token ids (role of kv_cache.cpp:24-29; the
    mixing function is this engine's own, hits are verified against stored ids anyway)."""
    h = _mix64(parent ^ 0x9E3779B97F4A7C15) ^ _mix64((salt + 0x2545F4914F6CDD1D) & _MASK)
    for t in tokens:
        h = _mix64(h ^ ((int(t) & 0xFFFFFFFF) + 0x9E3779B97F4A7C15 + ((h << 6) & _MASK) + (h >> 2)))
    return h if h != HASH_NONE else 1


class PoolError(RuntimeError):
    pass


class BlockPool:
    def __init__(self, num_blocks: int, block_size: int, enable_caching: bool = True):
        if num_blocks < 1 or block_size < 1:
            raise ValueError("BlockPool needs at least one block of at least one token")
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.caching = enable_caching
        self.ref = [0] * num_blocks
        self.hash = [HASH_NONE] * num_blocks
        self.tokens: List[Optional[Tuple[int, ...]]] = [None] * num_blocks
        self._prev = [-1] * num_blocks
        self._next = [-1] * num_blocks
        self._in_free = [False] * num_blocks
        self._head = -1
        self._tail = -1
        self.num_free = 0
        self._index: Dict[int, List[int]] = {}        # hash -> pages carrying it
        self.cache_queries = 0
        self.cache_hits = 0
        self.evictions = 0
        for b in range(num_blocks):
            self._push_back(b)

    # ---- free list -------------------------------------------------------------------
    def _remove(self, b: int) -> None:
        if not self._in_free[b]:
            return
        p, n = self._prev[b], self._next[b]
        if p >= 0:
            self._next[p] = n
        else:
            self._head = n
        if n >= 0:
            self._prev[n] = p
        else:
            self._tail = p
        self._prev[b] = self._next[b] = -1
        self._in_free[b] = False
        self.num_free -= 1

    def _push_front(self, b: int) -> None:
        self._prev[b] = -1
        self._next[b] = self._head
        if self._head >= 0:
            self._prev[self._head] = b
        else:
            self._tail = b
        self._head = b
        self._in_free[b] = True
        self.num_free += 1

    def _push_back(self, b: int) -> None:
        self._next[b] = -1
        self._prev[b] = self._tail
        if self._tail >= 0:
            self._next[self._tail] = b
        else:
            self._head = b
        self._tail = b
        self._in_free[b] = True
        self.num_free += 1

    def free_list(self) -> List[int]:
        out, b = [], self._head
        while b >= 0:
            out.append(b)
            b = self._next[b]
        return out

    # ---- prefix index ----------------------------------------------------------------
    def _evict_hash(self, b: int) -> None:
        h = self.hash[b]
        if h == HASH_NONE:
            return
        lst = self._index.get(h)
        if lst is not None:
            if b in lst:
                lst.remove(b)
            if not lst:
                del self._index[h]
        self.hash[b] = HASH_NONE
        self.tokens[b] = None
        self.evictions += 1

    @property
    def num_cached(self) -> int:
        return sum(len(v) for v in self._index.values())

    def get_cached_block(self, h: int, tokens: Sequence[int]) -> int:
        if not self.caching:
            return -1
        want = tuple(tokens)
        for b in self._index.get(h, ()):
            if self.tokens[b] == want:
                return b
        return -1

    def is_cached(self, b: int) -> bool:
        return self.hash[b] != HASH_NONE

    def cache_block(self, b: int, h: int, tokens: Sequence[int]) -> None:
        if not self.caching or self.hash[b] != HASH_NONE:
            return
        self.hash[b] = h
        self.tokens[b] = tuple(tokens)
        self._index.setdefault(h, []).append(b)

    def reset_prefix_cache(self) -> bool:
        if self.num_free != self.num_blocks:
            return False
        for b in range(self.num_blocks):
            self.hash[b] = HASH_NONE
            self.tokens[b] = None
        self._index.clear()
        return True

    # ---- references ------------------------------------------------------------------
    def touch(self, b: int) -> None:
        """Take a reference; a free page (kept only for its prefix) leaves the free list."""
        if self.ref[b] == 0:
            self._remove(b)
        self.ref[b] += 1

    def get_new_blocks(self, n: int) -> List[int]:
        if n > self.num_free:
            raise PoolError(f"BlockPool: out of blocks (asked {n}, free {self.num_free})")
        out = []
        for _ in range(n):
            b = self._head
            self._remove(b)
            if self.hash[b] != HASH_NONE:
                self._evict_hash(b)
            self.ref[b] = 1
            out.append(b)
        return out

    def free_blocks(self, blocks: Iterable[int]) -> None:
        uncached, cached = [], []
        for b in blocks:
            if self.ref[b] <= 0:
                raise PoolError(f"BlockPool: double free of block {b}")
            self.ref[b] -= 1
            if self.ref[b] == 0:
                if self.hash[b] == HASH_NONE or not self.caching:
                    uncached.append(b)
                else:
                    cached.append(b)
        for b in reversed(uncached):
            self._push_front(b)
        for b in cached:
            self._push_back(b)

    @property
    def usage(self) -> float:
        return 1.0 - self.num_free / self.num_blocks

    def check_invariants(self) -> None:
        """Every page is either referenced or on the free list, never both or neither."""
        on_list = self.free_list()
        if len(on_list) != len(set(on_list)):
            raise AssertionError("a page is on the free list twice")
        if len(on_list) != self.num_free:
            raise AssertionError(f"free list holds {len(on_list)} pages, counter says {self.num_free}")
        free_set = set(on_list)
        for b in range(self.num_blocks):
            if (self.ref[b] == 0) != (b in free_set):
                raise AssertionError(f"page {b}: ref {self.ref[b]}, on free list {b in free_set}")
            if self.ref[b] < 0:
                raise AssertionError(f"page {b} has negative ref {self.ref[b]}")
