"""The cache manager: pages per group of layers, a block table per request and group, prefix reuse, and
slots for per-request state of fixed size.

The manager is C++ (``include/iian_b200/cache_manager.h``; what it keeps of the reference and what is new
is said there); the classes here are handles on it.  Everything is host bookkeeping on page numbers; device
tensors live in ``iian_b200.cache.storage``.
"""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_uint64
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

from . import native
from .block_pool import HASH_NONE, BlockPool, PoolError, hash_block

__all__ = ["CacheManager", "PageGroup", "RequestCache", "StateSlots", "PoolError", "hash_block", "HASH_NONE"]


@dataclass(frozen=True)
class PageGroup:
    """Caches (by id) whose mixers have the same need and therefore share a block table."""

    name: str
    cache_ids: Tuple[int, ...]
    window: Optional[int]          # None: every key stays; n: a query sees itself and the n-1 keys before it
    num_blocks: int


class RequestCache:
    """What one request holds: per group the page of each logical block (-1 = not held), the chained hashes
    of its full pages, its state slot.  A handle on the native record; ``_owner`` is what keeps that record
    alive when it is not this object (a scheduler's request)."""

    __slots__ = ("_h", "_owner", "_n_groups", "__weakref__")

    def __init__(self, handle, n_groups: int, owner=None):
        self._h, self._n_groups, self._owner = handle, n_groups, owner

    def __del__(self):
        if getattr(self, "_owner", None) is None and getattr(self, "_h", None):
            try:
                native.lib().iian_rc_delete(self._h)
            except Exception:           # the interpreter is shutting down
                pass
            self._h = None

    def _get(self, what: int, g: int = 0) -> int:
        return native.lib().iian_rc_get(self._h, what, g)

    def table(self, g: int) -> List[int]:
        n = self._get(3, g)
        return list(native.lib().iian_rc_table(self._h, g)[:n]) if n > 0 else []

    tables = property(lambda self: [self.table(g) for g in range(self._n_groups)])
    committed = property(lambda self: [self._get(5, g) for g in range(self._n_groups)])
    state_slot = property(lambda self: self._get(0))
    epoch = property(lambda self: self._get(2))

    @property
    def hashes(self) -> List[int]:
        n = self._get(4)
        return list(native.lib().iian_rc_hashes(self._h)[:n]) if n > 0 else []

    @property
    def state_fresh(self) -> bool:
        return bool(self._get(1))

    @state_fresh.setter
    def state_fresh(self, v: bool) -> None:
        native.lib().iian_rc_set_state_fresh(self._h, int(bool(v)))

    def holds_pages(self) -> bool:
        return bool(self._get(6))


class StateSlots:
    """Fixed-size per-request state: slot numbers handed out at admission, taken back at the end."""

    def __init__(self, mgr):
        """``mgr``: the cache manager whose slots these are, or a number of slots for a set of its own."""
        if isinstance(mgr, int):
            mgr = CacheManager([PageGroup("none", (), None, 1)], 1, False, mgr)
        self._mgr = mgr

    def _call(self, what: int, arg: int = 0) -> int:
        out = c_int(0)
        native.check(native.lib().iian_cache_slots(self._mgr._h, what, arg, out))
        return out.value

    num_slots = property(lambda self: self._call(0))
    num_free = property(lambda self: self._call(1))

    def allot(self) -> int:
        return self._call(2)

    def release(self, slot: int) -> None:
        self._call(3, slot)


class CacheManager:
    def __init__(self, groups: Sequence[PageGroup], block_size: int, enable_prefix_caching: bool = True,
                 num_state_slots: int = 0):
        if block_size < 1:
            raise ValueError("block_size must be >= 1")
        self.groups = list(groups)
        self.block_size = block_size
        self.prefix_caching = enable_prefix_caching
        L = native.lib()
        windows, n = native.int_array([-1 if g.window is None else int(g.window) for g in self.groups])
        blocks, _ = native.int_array([int(g.num_blocks) for g in self.groups])
        self._h = L.iian_cache_new(windows, blocks, n, block_size, int(enable_prefix_caching), num_state_slots)
        if not self._h:
            raise ValueError(L.iian_host_last_error().decode())
        self.pools = [BlockPool(g.num_blocks, block_size, enable_prefix_caching, _handle=L.iian_cache_pool(self._h, i), _owner=self)
                      for i, g in enumerate(self.groups)]
        self.slots = StateSlots(self)

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                native.lib().iian_cache_delete(self._h)
            except Exception:           # the interpreter is shutting down
                pass
            self._h = None

    prefix_queries = property(lambda self: native.lib().iian_cache_counter(self._h, 0, 0))
    prefix_hits = property(lambda self: native.lib().iian_cache_counter(self._h, 1, 0))

    # ---- requests --------------------------------------------------------------------
    def new_request(self) -> RequestCache:
        return RequestCache(native.lib().iian_rc_new(self._h), len(self.groups))

    def allot_state(self, rc: RequestCache) -> bool:
        """Give the request a state slot (no-op if it has one).  False if none is free."""
        return bool(native.lib().iian_cache_allot_state(self._h, rc._h))

    # ---- geometry --------------------------------------------------------------------
    def first_needed_block(self, g: int, n_computed: int) -> int:
        """First logical block a group still needs once ``n_computed`` tokens are done: the next
        query sits at position ``n_computed`` and sees keys ``> n_computed - window``."""
        return native.lib().iian_cache_first_needed_block(self._h, g, n_computed)

    def blocks_for(self, n_tokens: int) -> int:
        return (n_tokens + self.block_size - 1) // self.block_size

    # ---- prefix reuse ----------------------------------------------------------------
    def update_hashes(self, rc: RequestCache, tokens: Sequence[int], salt: int = 0) -> None:
        """Extend the request's chained hashes to cover every full page of ``tokens``."""
        arr, n = native.i32_array(list(tokens))
        native.check(native.lib().iian_cache_update_hashes(self._h, rc._h, arr, n, salt & ((1 << 64) - 1)))

    def _table_buffers(self, cap: int):
        return (c_int * (len(self.groups) * max(cap, 1)))(), (c_int * len(self.groups))()

    def find_cached_prefix(self, tokens: Sequence[int], hashes: Sequence[int]) -> Tuple[int, List[List[int]]]:
        """Longest reusable prefix, in tokens (a multiple of the page size, at most ``len(tokens) - 1`` so
        that the last token is always computed for its logits), and per group the table to start from.
        Nothing is referenced yet."""
        arr, n = native.i32_array(list(tokens))
        hs = (c_uint64 * max(len(hashes), 1))(*hashes)
        cap = max(1, self.blocks_for(n))
        tables, lens = self._table_buffers(cap)
        found = native.lib().iian_cache_find_prefix(self._h, arr, n, hs, len(hashes), tables, lens, cap)
        if found < 0:
            native.check(2)
        return found, [list(tables[g * cap: g * cap + lens[g]]) for g in range(len(self.groups))]

    def commit(self, rc: RequestCache, tokens: Sequence[int], n_computed: int) -> None:
        """Offer the full pages covering ``tokens[:n_computed]`` to the prefix index."""
        arr, n = native.i32_array(list(tokens))
        native.check(native.lib().iian_cache_commit(self._h, rc._h, arr, n, n_computed))

    # ---- pages -----------------------------------------------------------------------
    def release_passed(self, rc: RequestCache, n_computed: int) -> int:
        """Give back pages that a group's window has passed.  Returns how many."""
        out = c_int(0)
        native.check(native.lib().iian_cache_release_passed(self._h, rc._h, n_computed, out))
        return out.value

    def allocate(self, rc: RequestCache, n_computed: int, n_new: int,
                 computed: Optional[List[List[int]]] = None) -> bool:
        """Make sure the request holds pages for tokens ``[0, n_computed + n_new)`` in every group (for a
        windowed group: from the first block its window still reaches).  Pages of a prefix hit
        (``computed``, from :meth:`find_cached_prefix`) are referenced and put first if the request holds
        nothing yet.  Either every group gets what it needs or nothing is taken and False is returned."""
        ok = c_int(0)
        if computed is None:
            native.check(native.lib().iian_cache_allocate(self._h, rc._h, n_computed, n_new, None, None, 0, ok))
        else:
            cap = max(1, max(len(t) for t in computed))
            tables, lens = self._table_buffers(cap)
            for g, t in enumerate(computed):
                lens[g] = len(t)
                tables[g * cap: g * cap + len(t)] = t
            native.check(native.lib().iian_cache_allocate(self._h, rc._h, n_computed, n_new, tables, lens, cap, ok))
        return bool(ok.value)

    def free(self, rc: RequestCache) -> None:
        """Give back everything the request holds: pages in reverse order, so that the tail of a chain is
        evicted before its head, and the state slot."""
        native.check(native.lib().iian_cache_free(self._h, rc._h))

    def slot_of(self, rc: RequestCache, g: int, token_idx: int) -> int:
        """Flat cache cell of a token: page * page size + offset (include/iian/kv_cache.h:135-137)."""
        out = c_longlong(0)
        native.check(native.lib().iian_cache_slot_of(self._h, rc._h, g, token_idx, out))
        return out.value

    # ---- figures ---------------------------------------------------------------------
    @property
    def usage(self) -> float:
        return native.lib().iian_cache_usage(self._h)

    def num_free(self, g: int = 0) -> int:
        return self.pools[g].num_free

    def check_invariants(self) -> None:
        if native.lib().iian_cache_check(self._h) != 0:
            raise AssertionError(native.lib().iian_host_last_error().decode())
