"""The cache manager in plain Python: the model that the native manager (include/iian_b200/cache_manager.h) is
tested against.

The cache manager: pages per group of layers, a block table per request and group,
prefix reuse, and slots for per-request state of fixed size.

The reference has one group (every layer shares one block table,
src/iian/kv_cache.cpp:156-169) and no fixed-size state; its per-request record is
``KVRequestState`` (include/iian/kv_cache.h:93-97) and its operations are
``get_computed_blocks`` (kv_cache.cpp:199-212), ``allocate_slots`` (:214-229, all or
nothing), ``cache_blocks`` (:231-238), ``free`` in reverse order (:240-246) and
``update_hashes`` (:190-197).  Those semantics are kept per group.  New here:

* several groups, each with a pool of its own; a group with a ``window`` needs only the
  last ``window`` keys, so pages the window has passed are given back while the request
  is still running ("free out-of-window blocks" is an open item in the reference,
  docs/ROADMAP.md:33);
* a prefix hit must be usable by every group: all leading pages for a group that needs all
  keys, the pages inside the window for a windowed one;
* :class:`StateSlots`: one fixed-size slot per running request for mixers that keep a
  summary instead of per-token entries.

Everything here is host bookkeeping on page numbers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from plain_block_pool import HASH_NONE, BlockPool, PoolError, hash_block


@dataclass(frozen=True)
class PageGroup:
    """Caches (by id) whose mixers have the same need and therefore share a block table."""

    name: str
    cache_ids: Tuple[int, ...]
    window: Optional[int]          # None: every key stays; n: a query sees itself and the n-1 keys before it
    num_blocks: int


@dataclass
class RequestCache:
    """What one request holds."""

    tables: List[List[int]] = field(default_factory=list)      # per group: page of logical block i, -1 = not held
    hashes: List[int] = field(default_factory=list)            # chained hashes of full pages of its tokens
    committed: List[int] = field(default_factory=list)         # per group: leading blocks offered to the prefix index
    state_slot: int = -1
    state_fresh: bool = False                                   # slot was just allotted and must start from zero
    epoch: int = 0                                              # bumped whenever a table changes other than by growing

    def holds_pages(self) -> bool:
        return any(any(p >= 0 for p in t) for t in self.tables)


class StateSlots:
    """Fixed-size per-request state: slot numbers handed out at admission, taken back at the end."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._held = [False] * num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allot(self) -> int:
        if not self._free:
            return -1
        s = self._free.pop()
        self._held[s] = True
        return s

    def release(self, slot: int) -> None:
        if slot < 0:
            return
        if not self._held[slot]:
            raise PoolError(f"StateSlots: slot {slot} released twice")
        self._held[slot] = False
        self._free.append(slot)


class CacheManager:
    def __init__(self, groups: Sequence[PageGroup], block_size: int, enable_prefix_caching: bool = True,
                 num_state_slots: int = 0):
        if block_size < 1:
            raise ValueError("block_size must be >= 1")
        self.groups = list(groups)
        self.block_size = block_size
        self.prefix_caching = enable_prefix_caching
        self.pools = [BlockPool(g.num_blocks, block_size, enable_prefix_caching) for g in self.groups]
        self.slots = StateSlots(num_state_slots)
        self.prefix_queries = 0        # pages asked for / found, as in kv_cache.h:86
        self.prefix_hits = 0

    # ---- requests --------------------------------------------------------------------
    def new_request(self) -> RequestCache:
        n = len(self.groups)
        return RequestCache(tables=[[] for _ in range(n)], committed=[0] * n)

    def allot_state(self, rc: RequestCache) -> bool:
        """Give the request a state slot (no-op if it has one).  False if none is free."""
        if rc.state_slot >= 0:
            return True
        if self.slots.num_slots == 0:
            return True
        s = self.slots.allot()
        if s < 0:
            return False
        rc.state_slot = s
        rc.state_fresh = True
        return True

    # ---- geometry --------------------------------------------------------------------
    def first_needed_block(self, g: int, n_computed: int) -> int:
        """First logical block a group still needs once ``n_computed`` tokens are done: the next
        query sits at position ``n_computed`` and sees keys ``> n_computed - window``."""
        w = self.groups[g].window
        if w is None:
            return 0
        return max(0, n_computed - w + 1) // self.block_size

    def blocks_for(self, n_tokens: int) -> int:
        return (n_tokens + self.block_size - 1) // self.block_size

    # ---- prefix reuse ----------------------------------------------------------------
    def update_hashes(self, hashes: List[int], tokens: Sequence[int], salt: int = 0) -> None:
        bs = self.block_size
        n_full = len(tokens) // bs
        while len(hashes) < n_full:
            i = len(hashes)
            parent = HASH_NONE if i == 0 else hashes[i - 1]
            hashes.append(hash_block(parent, tokens[i * bs:(i + 1) * bs], salt))

    def find_cached_prefix(self, tokens: Sequence[int], hashes: Sequence[int]) -> Tuple[int, List[List[int]]]:
        """Longest reusable prefix, in tokens (a multiple of the page size, at most
        ``len(tokens) - 1`` so that the last token is always computed for its logits), and
        per group the table to start from.  Nothing is referenced yet."""
        empty = [[] for _ in self.groups]
        if not self.prefix_caching or len(tokens) < 2:
            return 0, empty
        bs = self.block_size
        max_blocks = min((len(tokens) - 1) // bs, len(hashes))
        found: List[List[int]] = [[] for _ in self.groups]
        for g, pool in enumerate(self.pools):
            for i in range(max_blocks):
                found[g].append(pool.get_cached_block(hashes[i], tokens[i * bs:(i + 1) * bs]))
        n = max_blocks
        for g, grp in enumerate(self.groups):
            if grp.window is None:
                k = 0
                while k < n and found[g][k] >= 0:
                    k += 1
                n = k
        while n > 0:
            ok = True
            for g, grp in enumerate(self.groups):
                if grp.window is None:
                    continue
                first = self.first_needed_block(g, n * bs)
                if any(found[g][i] < 0 for i in range(first, n)):
                    ok = False
                    break
            if ok:
                break
            n -= 1
        if n == 0:
            return 0, empty
        tables = []
        for g, grp in enumerate(self.groups):
            first = self.first_needed_block(g, n * bs)
            tables.append([-1] * first + [found[g][i] for i in range(first, n)])
        return n * bs, tables

    def commit(self, rc: RequestCache, tokens: Sequence[int], n_computed: int) -> None:
        """Offer the full pages covering ``tokens[:n_computed]`` to the prefix index."""
        if not self.prefix_caching:
            return
        bs = self.block_size
        n_full = min(min(n_computed, len(tokens)) // bs, len(rc.hashes))
        for g, pool in enumerate(self.pools):
            table = rc.tables[g]
            for i in range(rc.committed[g], min(n_full, len(table))):
                if table[i] >= 0:
                    pool.cache_block(table[i], rc.hashes[i], tokens[i * bs:(i + 1) * bs])
            rc.committed[g] = max(rc.committed[g], min(n_full, len(table)))

    # ---- pages -----------------------------------------------------------------------
    def release_passed(self, rc: RequestCache, n_computed: int) -> int:
        """Give back pages that a group's window has passed.  Returns how many."""
        released = 0
        for g, pool in enumerate(self.pools):
            if self.groups[g].window is None:
                continue
            table = rc.tables[g]
            first = min(self.first_needed_block(g, n_computed), len(table))
            gone = [i for i in range(first) if table[i] >= 0]
            if gone:
                pool.free_blocks([table[i] for i in reversed(gone)])
                for i in gone:
                    table[i] = -1
                released += len(gone)
        if released:
            rc.epoch += 1
        return released

    def allocate(self, rc: RequestCache, n_computed: int, n_new: int,
                 computed: Optional[List[List[int]]] = None) -> bool:
        """Make sure the request holds pages for tokens ``[0, n_computed + n_new)`` in every
        group (for a windowed group: from the first block its window still reaches).  Pages
        of a prefix hit (``computed``, from :meth:`find_cached_prefix`) are referenced and put
        first if the request holds nothing yet.  Either every group gets what it needs or
        nothing is taken and False is returned."""
        self.release_passed(rc, n_computed)
        need_total = self.blocks_for(n_computed + n_new)
        plans = []
        for g, pool in enumerate(self.pools):
            table = rc.tables[g]
            use_computed = computed is not None and not table and bool(computed[g])
            have = len(computed[g]) if use_computed else len(table)
            n_fresh = max(0, need_total - have)
            n_touch_free = 0
            if use_computed:
                n_touch_free = sum(1 for p in computed[g] if p >= 0 and pool.ref[p] == 0)
            if n_fresh + n_touch_free > pool.num_free:
                return False
            plans.append((use_computed, n_fresh))
        for g, pool in enumerate(self.pools):
            use_computed, n_fresh = plans[g]
            table = rc.tables[g]
            if use_computed:
                for p in computed[g]:
                    if p >= 0:
                        pool.touch(p)
                    table.append(p)
                rc.committed[g] = len(table)
            if n_fresh:
                table.extend(pool.get_new_blocks(n_fresh))
        return True

    def free(self, rc: RequestCache) -> None:
        """Give back everything the request holds: pages in reverse order, so that the tail of
        a chain is evicted before its head, and the state slot."""
        for g, pool in enumerate(self.pools):
            table = rc.tables[g]
            held = [p for p in reversed(table) if p >= 0]
            if held:
                pool.free_blocks(held)
            table.clear()
            rc.committed[g] = 0
        rc.epoch += 1
        if rc.state_slot >= 0:
            self.slots.release(rc.state_slot)
            rc.state_slot = -1
            rc.state_fresh = False

    def slot_of(self, rc: RequestCache, g: int, token_idx: int) -> int:
        """Flat cache cell of a token: page * page size + offset (include/iian/kv_cache.h:135-137)."""
        page = rc.tables[g][token_idx // self.block_size]
        if page < 0:
            raise PoolError(f"token {token_idx} lies in a page that was given back")
        return page * self.block_size + token_idx % self.block_size

    # ---- figures ---------------------------------------------------------------------
    @property
    def usage(self) -> float:
        return max(p.usage for p in self.pools) if self.pools else 0.0

    def num_free(self, g: int = 0) -> int:
        return self.pools[g].num_free

    def check_invariants(self) -> None:
        for p in self.pools:
            p.check_invariants()
