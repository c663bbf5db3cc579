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
    finished: bool = False
    finish_reason: FinishReason = FinishReason.NONE
    stop_reason: str = ""
    error: str = ""
    n_prompt_tokens: int = 0
    n_output_tokens: int = 0
    n_cached_tokens: int = 0


@dataclass
class Request:
    id: int
    tokens: List[int]                       # prompt + generated
    n_prompt: int
    params: SamplingParams
    priority: int = 0
    cache_salt: int = 0
    arrival: float = field(default_factory=time.monotonic)
    status: RequestStatus = RequestStatus.WAITING
    finish_reason: FinishReason = FinishReason.NONE
    stop_reason: str = ""
    error: str = ""
    num_computed_tokens: int = 0            # catches up with len(tokens) (request.h:74)
    num_cached_tokens: int = 0              # prefix hit at first admission
    num_preemptions: int = 0
    cache: Optional[RequestCache] = None
    seed: int = 0                           # sampling stream of this request
    outputs: List[OutputChunk] = field(default_factory=list)
    pending_tokens: List[int] = field(default_factory=list)
    t_first_token: float = 0.0
    t_last_token: float = 0.0
    t_finished: float = 0.0

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
        return self.tokens[self.n_prompt:]
