"""A pool of fixed-size cache pages with reference counts, a free list and a prefix index.

The pool itself is C++ (``include/iian_b200/block_pool.h``, after the reference's ``BlockPool``,
include/iian/kv_cache.h:40-90 and src/iian/kv_cache.cpp:34-132); this class is a handle on it.  No device
memory is touched here; pages are numbers.
"""
from __future__ import annotations

from ctypes import c_int
from typing import Iterable, List, Sequence

from . import native
from .native import PoolError

HASH_NONE = 0

__all__ = ["BlockPool", "PoolError", "hash_block", "HASH_NONE"]


def hash_block(parent: int, tokens: Sequence[int], salt: int = 0) -> int:
    """Chained 64-bit hash of one full page of token ids (role of kv_cache.cpp:24-29)."""
    arr, n = native.i32_array([int(t) for t in tokens])
    return native.lib().iian_hash_block(parent & ((1 << 64) - 1), arr, n, salt & ((1 << 64) - 1))


class _PerPage:
    """``pool.ref[b]`` / ``pool.hash[b]``: read one page's field from the native pool."""

    def __init__(self, pool: "BlockPool", what: str):
        self._pool, self._what = pool, what

    def __getitem__(self, b: int) -> int:
        L = native.lib()
        if not 0 <= b < self._pool.num_blocks:
            raise IndexError(b)
        if self._what == "hash":
            return L.iian_pool_hash(self._pool._h, b)
        return L.iian_pool_get(self._pool._h, 5, b)

    def __len__(self) -> int:
        return self._pool.num_blocks

    def __iter__(self):
        return (self[b] for b in range(len(self)))

    def __eq__(self, other) -> bool:
        return list(self) == list(other)


class BlockPool:
    def __init__(self, num_blocks: int, block_size: int, enable_caching: bool = True, _handle=None, _owner=None):
        if num_blocks < 1 or block_size < 1:
            raise ValueError("BlockPool needs at least one block of at least one token")
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.caching = enable_caching
        self._owner = _owner           # a pool that belongs to a cache manager lives as long as the manager
        self._h = _handle if _handle is not None else native.lib().iian_pool_new(num_blocks, block_size, int(enable_caching))
        self.ref = _PerPage(self, "ref")
        self.hash = _PerPage(self, "hash")

    def __del__(self):
        if getattr(self, "_owner", None) is None and getattr(self, "_h", None):
            try:
                native.lib().iian_pool_delete(self._h)
            except Exception:           # the interpreter is shutting down
                pass
            self._h = None

    def _get(self, what: int) -> int:
        return native.lib().iian_pool_get(self._h, what, 0)

    num_free = property(lambda self: self._get(3))
    num_cached = property(lambda self: self._get(4))
    evictions = property(lambda self: self._get(7))
    cache_queries = property(lambda self: self._get(8))
    cache_hits = property(lambda self: self._get(9))
    usage = property(lambda self: 1.0 - self.num_free / self.num_blocks)

    def free_list(self) -> List[int]:
        buf = (c_int * self.num_blocks)()
        n = native.lib().iian_pool_free_list(self._h, buf, self.num_blocks)
        return list(buf[:n])

    def get_cached_block(self, h: int, tokens: Sequence[int]) -> int:
        arr, n = native.i32_array(list(tokens))
        return native.lib().iian_pool_get_cached_block(self._h, h, arr, n)

    def is_cached(self, b: int) -> bool:
        return bool(native.lib().iian_pool_get(self._h, 6, b))

    def cache_block(self, b: int, h: int, tokens: Sequence[int]) -> None:
        arr, n = native.i32_array(list(tokens))
        native.check(native.lib().iian_pool_cache_block(self._h, b, h, arr, n))

    def reset_prefix_cache(self) -> bool:
        return bool(native.lib().iian_pool_reset_prefix_cache(self._h))

    def touch(self, b: int) -> None:
        """Take a reference; a free page (kept only for its prefix) leaves the free list."""
        native.check(native.lib().iian_pool_touch(self._h, b))

    def get_new_blocks(self, n: int) -> List[int]:
        buf = (c_int * max(n, 1))()
        native.check(native.lib().iian_pool_get_new_blocks(self._h, n, buf))
        return list(buf[:n])

    def free_blocks(self, blocks: Iterable[int]) -> None:
        arr, n = native.int_array(list(blocks))
        native.check(native.lib().iian_pool_free_blocks(self._h, arr, n))

    def check_invariants(self) -> None:
        """Every page is either referenced or on the free list, never both or neither."""
        code = native.lib().iian_pool_check(self._h)
        if code != 0:
            raise AssertionError(native.lib().iian_host_last_error().decode())
