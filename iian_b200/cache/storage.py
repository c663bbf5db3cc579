"""Device memory of the caches.

One tensor per page group holds the keys and values of all its caches:
``[caches, 2 (K, V), pages, kv_heads, page_size, head_dim]`` in the activation dtype, so that one
(page, head) tile of K or V is contiguous.  The reference stores token-major rows
``[n_embd_gqa, n_cells]`` per layer (src/iian/kv_cache.cpp:163-164); the cell numbering
(page * page_size + offset, include/iian/kv_cache.h:135-137) is the same.

Fixed-size state: one tensor ``[slots, *shape]`` per cache that asked for it, zeroed when a slot is
handed to a new request.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import KVNeed, StateNeed
from .manager import PageGroup


@dataclass
class KVView:
    group: int            # index of the page group (selects block table and slots in the step context)
    k: torch.Tensor       # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor


@dataclass
class StateView:
    state: torch.Tensor   # [slots, *shape]


def plan_groups(needs: Dict[int, object], capacity_tokens: int, block_size: int,
                window_tokens: Optional[int] = None) -> Tuple[List[PageGroup], List[KVNeed]]:
    """Group caches with the same KV need.  ``capacity_tokens`` sizes a group that keeps all keys;
    a windowed group gets ``window_tokens`` if given (else the same)."""
    by_need: Dict[KVNeed, List[int]] = {}
    for cid in sorted(needs):
        need = needs[cid]
        if isinstance(need, KVNeed):
            by_need.setdefault(need, []).append(cid)
    groups, kinds = [], []
    for need, cids in by_need.items():
        tokens = capacity_tokens if need.window is None or window_tokens is None else min(capacity_tokens, window_tokens)
        n_blocks = max(1, (tokens + block_size - 1) // block_size)
        name = f"kv{need.num_kv_heads}x{need.head_dim}" + (f"w{need.window}" if need.window else "")
        groups.append(PageGroup(name=name, cache_ids=tuple(cids), window=need.window, num_blocks=n_blocks))
        kinds.append(need)
    return groups, kinds


class CacheStorage:
    def __init__(self, needs: Dict[int, object], groups: Sequence[PageGroup], kinds: Sequence[KVNeed],
                 block_size: int, num_state_slots: int, dtype: torch.dtype, device: torch.device):
        self.groups = list(groups)
        self.block_size = block_size
        self.dtype = dtype
        self.device = device
        self._views: Dict[int, object] = {}
        self.kv: List[torch.Tensor] = []
        self.states: Dict[int, torch.Tensor] = {}
        self.bytes = 0
        for g, (grp, need) in enumerate(zip(groups, kinds)):
            t = torch.zeros((len(grp.cache_ids), 2, grp.num_blocks, need.num_kv_heads, block_size, need.head_dim),
                            dtype=dtype, device=device)
            self.kv.append(t)
            self.bytes += t.numel() * t.element_size()
            for i, cid in enumerate(grp.cache_ids):
                self._views[cid] = KVView(group=g, k=t[i, 0], v=t[i, 1])
        for cid, need in needs.items():
            if isinstance(need, StateNeed):
                t = torch.zeros((max(1, num_state_slots),) + tuple(need.shape), dtype=need.dtype, device=device)
                self.states[cid] = t
                self.bytes += t.numel() * t.element_size()
                self._views[cid] = StateView(state=t)

    def view(self, cache_id: int):
        return self._views.get(cache_id)

    def zero_state(self, slots: Sequence[int]) -> None:
        if not slots or not self.states:
            return
        idx = torch.tensor(list(slots), dtype=torch.long, device=self.device)
        for t in self.states.values():
            t.index_fill_(0, idx, 0)
