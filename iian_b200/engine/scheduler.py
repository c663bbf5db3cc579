"""The scheduler: which requests run in the next step, and how many tokens of each.

The algorithm (the reference's, src/iian/scheduler.cpp:84-171) is C++: ``include/iian_b200/scheduler.h`` says
what it does; this class is a handle on it that maps the native records back to the ``Request`` objects of
the engine.
"""
from __future__ import annotations

from ctypes import c_int, c_void_p
from dataclasses import dataclass, field
from typing import Dict, List

from ..cache import native
from ..cache.manager import CacheManager
from ..config.engine import SchedulerConfig
from .request import Request, RequestStatus


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
        self._h = native.lib().iian_sched_new(cache._h, cfg.max_num_seqs, cfg.max_num_batched_tokens,
                                              cfg.long_prefill_token_threshold, int(cfg.enable_chunked_prefill),
                                              int(cfg.policy == "priority"))
        if not self._h:
            raise ValueError(native.lib().iian_host_last_error().decode())
        self._by_handle: Dict[int, Request] = {}       # native record -> request; also keeps the requests alive
        self._cap = 0
        self._grow(max(64, cfg.max_num_seqs + 8))

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                native.lib().iian_sched_delete(self._h)
            except Exception:           # the interpreter is shutting down
                pass
            self._h = None

    def _grow(self, cap: int) -> None:
        self._cap = cap
        self._reqs, self._pre = (c_void_p * cap)(), (c_void_p * cap)()
        self._n_new, self._resumed = (c_int * cap)(), (c_int * cap)()

    # ---- queues ----------------------------------------------------------------------
    def add_request(self, req: Request) -> None:
        self._by_handle[req._h] = req
        native.check(native.lib().iian_sched_add(self._h, req._h))
        if len(self._by_handle) + 8 > self._cap:
            self._grow(2 * self._cap)

    def _queue(self, which: int) -> List[Request]:
        n = native.lib().iian_sched_queue(self._h, which, self._reqs, self._cap)
        return [self._by_handle[self._reqs[i]] for i in range(n)]

    waiting = property(lambda self: self._queue(0))
    running = property(lambda self: self._queue(1))
    num_preemptions = property(lambda self: native.lib().iian_sched_num_preemptions(self._h))

    def all_requests(self) -> List[Request]:
        return self.running + self.waiting

    @property
    def has_requests(self) -> bool:
        return bool(self._by_handle)

    def finish_request(self, req: Request, status: RequestStatus) -> None:
        native.check(native.lib().iian_sched_finish(self._h, req._h, int(status)))
        self._by_handle.pop(req._h, None)

    # ---- one step --------------------------------------------------------------------
    def schedule(self) -> SchedulerOutput:
        n_s, n_p, total = c_int(0), c_int(0), c_int(0)
        native.check(native.lib().iian_sched_schedule(self._h, self._reqs, self._n_new, self._resumed, self._cap, n_s,
                                                      self._pre, n_p, total))
        out = SchedulerOutput(total_tokens=total.value)
        by = self._by_handle
        for i in range(n_s.value):
            out.scheduled.append(ScheduledRequest(by[self._reqs[i]], self._n_new[i], bool(self._resumed[i])))
        for i in range(n_p.value):
            out.preempted.append(by[self._pre[i]])
        return out

    def update_after_step(self, out: SchedulerOutput) -> None:
        """Advance the computed counts of the step that ran the last ``schedule()`` and offer its full pages to
        the prefix index."""
        native.check(native.lib().iian_sched_update(self._h))
