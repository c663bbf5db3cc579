"""The scheduler in plain Python: the model that the native scheduler (include/iian_b200/scheduler.h) is
tested against.

The scheduler: which requests run in the next step, and how many tokens of each.

The algorithm is the reference's (src/iian/scheduler.cpp:84-160, described in
docs/ARCHITECTURE.md:129-145):

* a request has ``num_computed_tokens`` and every step schedules work so that it catches up
  with ``len(tokens)``; there are no separate prefill and decode phases;
* phase 1, running requests in order: ``n_new = min(remaining, long-prefill cap, budget)``;
  pages are allocated for ``computed + n_new`` tokens (scheduler.cpp:89-124);
* when pages run out, the LAST running request is preempted (its pages freed, its computed
  count set to zero, itself put back at the front of the waiting queue) and the allocation is
  tried again; a victim that was already scheduled in this step gets its tokens refunded; if
  the victim is the request itself, scheduling stops (scheduler.cpp:105-118, :70-82);
* phase 2, admission from the waiting queue, only in a step that preempted nobody: look up the
  cached prefix, allocate, never preempt on behalf of a waiting request (scheduler.cpp:126-158);
* after the step the computed counts advance and full pages are offered to the prefix
  index (scheduler.cpp:162-171).

No speculative tokens.  New here: a request also needs a state slot before it is admitted.
"""
from __future__ import annotations

import bisect
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional

from plain_cache_manager import CacheManager, RequestCache

from iian_b200.config.engine import SchedulerConfig
from iian_b200.engine.request import RequestStatus


@dataclass
class Request:
    """What the scheduler needs of a request."""
    id: int
    tokens: List[int]
    priority: int = 0
    cache_salt: int = 0
    arrival: float = 0.0
    status: RequestStatus = RequestStatus.WAITING
    num_computed_tokens: int = 0
    num_cached_tokens: int = 0
    num_preemptions: int = 0
    cache: Optional[RequestCache] = None

    @property
    def n_tokens(self) -> int:
        return len(self.tokens)

    @property
    def is_finished(self) -> bool:
        return self.status > RequestStatus.PREEMPTED


@dataclass
class ScheduledRequest:
    req: Request
    n_new_tokens: int
    resumed: bool = False


@dataclass
class SchedulerOutput:
    scheduled: List[ScheduledRequest] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    total_tokens: int = 0


class Scheduler:
    def __init__(self, cfg: SchedulerConfig, cache: CacheManager):
        cfg.validate()
        self.cfg = cfg
        self.cache = cache
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.num_preemptions = 0

    # ---- queues ----------------------------------------------------------------------
    def add_request(self, req: Request) -> None:
        req.status = RequestStatus.WAITING
        if req.cache is None:
            req.cache = self.cache.new_request()
        self._enqueue(req)

    def _enqueue(self, req: Request) -> None:
        if self.cfg.policy == "priority":
            keys = [(r.priority, r.arrival) for r in self.waiting]
            pos = bisect.bisect_right(keys, (req.priority, req.arrival))
            self.waiting.insert(pos, req)
        else:
            self.waiting.append(req)

    def all_requests(self) -> List[Request]:
        return list(self.running) + list(self.waiting)

    @property
    def has_requests(self) -> bool:
        return bool(self.waiting) or bool(self.running)

    def finish_request(self, req: Request, status: RequestStatus) -> None:
        req.status = status
        if req.cache is not None:
            self.cache.free(req.cache)
        if req in self.running:
            self.running.remove(req)
        elif req in self.waiting:
            self.waiting.remove(req)

    def _preempt(self, req: Request) -> None:
        self.cache.free(req.cache)
        req.status = RequestStatus.PREEMPTED
        req.num_computed_tokens = 0
        req.num_preemptions += 1
        self.num_preemptions += 1
        self.running.remove(req)
        if self.cfg.policy == "priority":
            self._enqueue(req)
        else:
            self.waiting.appendleft(req)

    # ---- one step --------------------------------------------------------------------
    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput()
        budget = self.cfg.max_num_batched_tokens
        cap = self.cfg.long_prefill_token_threshold

        idx = 0
        while idx < len(self.running) and budget > 0:
            req = self.running[idx]
            n_new = req.n_tokens - req.num_computed_tokens
            if cap > 0:
                n_new = min(n_new, cap)
            n_new = min(n_new, budget)
            if n_new == 0:
                idx += 1
                continue
            ok = True
            while not self.cache.allocate(req.cache, req.num_computed_tokens, n_new):
                victim = self.running[-1]
                if victim is req:
                    self._preempt(req)
                    out.preempted.append(req)
                    ok = False
                    break
                for s in out.scheduled:
                    if s.req is victim:
                        budget += s.n_new_tokens
                        out.total_tokens -= s.n_new_tokens
                        out.scheduled.remove(s)
                        break
                self._preempt(victim)
                out.preempted.append(victim)
            if not ok:
                break
            out.scheduled.append(ScheduledRequest(req, n_new, False))
            out.total_tokens += n_new
            budget -= n_new
            idx += 1

        if not out.preempted:
            while self.waiting and budget > 0 and len(self.running) < self.cfg.max_num_seqs:
                req = self.waiting[0]
                computed = None
                n_computed = req.num_computed_tokens
                if n_computed == 0:
                    self.cache.update_hashes(req.cache.hashes, req.tokens, req.cache_salt)
                    n_computed, computed = self.cache.find_cached_prefix(req.tokens, req.cache.hashes)
                    self.cache.prefix_queries += len(req.tokens) // self.cache.block_size
                    self.cache.prefix_hits += n_computed // self.cache.block_size
                n_new = req.n_tokens - n_computed
                if cap > 0:
                    n_new = min(n_new, cap)
                if not self.cfg.enable_chunked_prefill and n_new > budget:
                    break
                n_new = min(n_new, budget)
                if n_new == 0:
                    break
                if not self.cache.allot_state(req.cache):
                    break
                if not self.cache.allocate(req.cache, n_computed, n_new, computed):
                    self.cache.free(req.cache)      # holds no pages; gives the state slot back
                    break
                self.waiting.popleft()
                resumed = req.status == RequestStatus.PREEMPTED
                req.status = RequestStatus.RUNNING
                req.num_computed_tokens = n_computed
                if not resumed:
                    req.num_cached_tokens = n_computed
                self.running.append(req)
                out.scheduled.append(ScheduledRequest(req, n_new, resumed))
                out.total_tokens += n_new
                budget -= n_new
        return out

    def update_after_step(self, out: SchedulerOutput) -> None:
        for s in out.scheduled:
            r = s.req
            if r.is_finished:
                continue
            r.num_computed_tokens += s.n_new_tokens
            self.cache.update_hashes(r.cache.hashes, r.tokens, r.cache_salt)
            self.cache.commit(r.cache, r.tokens, min(r.num_computed_tokens, r.n_tokens))
