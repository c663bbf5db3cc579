"""Per-request state and the chunks handed back to the submitter.

Fields follow the reference's ``Request`` / ``OutputChunk`` / ``RequestStatus`` /
``FinishReason`` (include/iian/request.h:21-39, :64-109) without the text, grammar,
embedding and speculative-decoding members.
"""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import List, Optional

from ctypes import c_int32

from ..cache import native
from ..cache.manager import RequestCache
from ..sampling.params import SamplingParams


class RequestStatus(enum.IntEnum):
    # ordering matters: finished states compare greater than PREEMPTED (request.h:20-21)
    WAITING = 0
    RUNNING = 1
    PREEMPTED = 2
    FINISHED_STOPPED = 3
    FINISHED_LENGTH = 4
    FINISHED_ABORTED = 5
    FINISHED_ERROR = 6


class FinishReason(enum.Enum):
    NONE = ""
    STOP = "stop"
    LENGTH = "length"
    ABORT = "abort"
    ERROR = "error"


@dataclass
class OutputChunk:
    tokens: List[int] = field(default_factory=list)
    logprobs: List = field(default_factory=list)      # parallel to tokens, if asked for: (logprob, [(id, logprob)])
    finished: bool = False
    finish_reason: FinishReason = FinishReason.NONE
    stop_reason: str = ""
    error: str = ""
    n_prompt_tokens: int = 0
    n_output_tokens: int = 0
    n_cached_tokens: int = 0


class _Tokens(list):
    """A request's token ids.  The scheduler's native record keeps a copy (it hashes pages of tokens and counts
    them), so what is appended here is appended there too."""

    __slots__ = ("_req",)

    def append(self, tok) -> None:
        list.append(self, tok)
        if self._req is not None:
            self._req._mirror([tok])

    def extend(self, toks) -> None:
        toks = list(toks)
        list.extend(self, toks)
        if self._req is not None:
            self._req._mirror(toks)


_GET = {"status": 0, "num_computed_tokens": 1, "num_cached_tokens": 2, "num_preemptions": 3}


class Request:
    """One request.  What the scheduler works with (tokens, status, computed / cached counts, preemptions, the
    cache record) lives in the native runtime (``include/iian_b200/scheduler.h: SchedRequest``); sampling
    parameters, outputs and times stay here."""

    def __init__(self, id: int, tokens: List[int], n_prompt: int, params: SamplingParams, priority: int = 0,
                 cache_salt: int = 0, arrival: Optional[float] = None, seed: int = 0):
        self.id = id
        self.n_prompt = n_prompt
        self.params = params
        self.priority = priority
        self.cache_salt = cache_salt
        self.arrival = time.monotonic() if arrival is None else arrival
        self.finish_reason = FinishReason.NONE
        self.stop_reason = ""
        self.error = ""
        self.seed = seed
        self.outputs: List[OutputChunk] = []
        self.pending_tokens: List[int] = []
        self.pending_logprobs: List = []
        self.logprobs: List = []                     # of all output tokens so far, if asked for
        self.t_first_token = self.t_last_token = self.t_finished = 0.0
        self.tokens = _Tokens(int(t) for t in tokens)       # prompt + generated
        self.tokens._req = None
        arr = (c_int32 * max(len(self.tokens), 1))(*self.tokens)
        self._h = native.lib().iian_req_new(id, arr, len(self.tokens), priority, float(self.arrival), cache_salt & ((1 << 64) - 1))
        self.tokens._req = self
        self._cache: Optional[RequestCache] = None
        self._cache_handle = None

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                native.lib().iian_req_delete(self._h)
            except Exception:           # the interpreter is shutting down
                pass
            self._h = None

    def _mirror(self, toks) -> None:
        arr = (c_int32 * len(toks))(*[int(t) for t in toks])
        native.lib().iian_req_append(self._h, arr, len(toks))

    def _native(self, what: int) -> int:
        return native.lib().iian_req_get(self._h, what)

    def _set_native(self, what: int, value: int) -> None:
        native.lib().iian_req_set(self._h, what, int(value))

    status = property(lambda self: RequestStatus(self._native(0)), lambda self, v: self._set_native(0, int(v)))
    num_computed_tokens = property(lambda self: self._native(1), lambda self, v: self._set_native(1, v))   # catches up with len(tokens) (request.h:74)
    num_cached_tokens = property(lambda self: self._native(2), lambda self, v: self._set_native(2, v))     # prefix hit at first admission
    num_preemptions = property(lambda self: self._native(3), lambda self, v: self._set_native(3, v))

    @property
    def cache(self) -> Optional[RequestCache]:
        """The request's cache record (None until a scheduler has taken the request)."""
        h = native.lib().iian_req_cache(self._h)
        if not h:
            return None
        if self._cache is None or self._cache_handle != h:
            n_groups = native.lib().iian_rc_get(h, 7, 0)
            self._cache = RequestCache(h, n_groups, owner=self)
            self._cache_handle = h
        return self._cache

    @cache.setter
    def cache(self, rc: Optional[RequestCache]) -> None:
        """Hand a cache record made with ``CacheManager.new_request`` to the request, which owns it from then on."""
        if rc is None:
            return
        native.lib().iian_req_adopt_cache(self._h, rc._h)
        rc._owner = self
        self._cache, self._cache_handle = rc, rc._h

    @property
    def n_tokens(self) -> int:
        return len(self.tokens)

    @property
    def n_output(self) -> int:
        return len(self.tokens) - self.n_prompt

    @property
    def is_finished(self) -> bool:
        return self.status > RequestStatus.PREEMPTED

    @property
    def output_tokens(self) -> List[int]:
        return list(self.tokens[self.n_prompt:])
