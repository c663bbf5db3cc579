"""Sampling parameters.

Names, defaults and validation follow ``SamplingParams`` of the reference
(include/iian/sampling.h:15-46, src/iian/sampler.cpp:13-28).  Penalties, logit bias, allowed
or bad words, logprobs, stop strings and grammars need token history or a tokenizer on the
sampling path and are not part of this engine.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class SamplingParams:
    temperature: float = 1.0          # < 1e-5 -> greedy (sampling.h:44)
    top_p: float = 1.0
    top_k: int = 0                    # 0 or -1 -> off
    min_p: float = 0.0
    seed: Optional[int] = None        # None -> engine seed + id * golden ratio (src/iian/engine.cpp:302)
    max_tokens: int = -1              # -1 -> until the context is full
    min_tokens: int = 0
    ignore_eos: bool = False
    stop_token_ids: List[int] = field(default_factory=list)

    @property
    def is_greedy(self) -> bool:
        return self.temperature < 1e-5

    def validate(self, n_vocab: int) -> None:
        if self.temperature < 0.0:
            raise ValueError("temperature must be >= 0")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < -1:
            raise ValueError("top_k must be -1, 0 or positive")
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError("min_p must be in [0, 1]")
        if self.max_tokens < -1 or self.max_tokens == 0:
            raise ValueError("max_tokens must be >= 1")
        if self.min_tokens < 0:
            raise ValueError("min_tokens must be >= 0")
        if self.max_tokens > 0 and self.min_tokens > self.max_tokens:
            raise ValueError("min_tokens must be <= max_tokens")
        for t in self.stop_token_ids:
            if t < 0 or t >= n_vocab:
                raise ValueError(f"stop_token_ids out of range: {t}")
