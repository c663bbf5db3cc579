"""Sampling parameters.

Names, defaults and validation follow ``SamplingParams`` of the reference
(include/iian/sampling.h:15-46, src/iian/sampler.cpp:13-28), the logits processors included: allowed ids, logit
bias, bad words and the presence / frequency / repetition penalties (sampler.cpp:72-109).  Log-probabilities are those of the raw
distribution (sampler.cpp:63-70, 174-182).  Stop strings and grammars need text and are not part of this engine.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional


@dataclass
class SamplingParams:
    temperature: float = 1.0          # < 1e-5 -> greedy (sampling.h:44)
    top_p: float = 1.0
    top_k: int = 0                    # 0 or -1 -> off
    min_p: float = 0.0
    presence_penalty: float = 0.0     # subtracted once from a token that was produced (within the window)
    frequency_penalty: float = 0.0    # subtracted once per time it was produced
    repetition_penalty: float = 1.0   # divides positive, multiplies negative logits of produced and prompt tokens
    repetition_last_n: int = -1       # window of output tokens the counts are taken over (-1 = all)
    seed: Optional[int] = None        # None -> engine seed + id * golden ratio (src/iian/engine.cpp:302)
    max_tokens: int = -1              # -1 -> until the context is full
    min_tokens: int = 0
    ignore_eos: bool = False
    stop_token_ids: List[int] = field(default_factory=list)
    logprobs: int = -1                # -1 none, 0 the produced token only, k: the k most likely tokens as well (<= 20)
    logit_bias: Dict[int, float] = field(default_factory=dict)
    allowed_token_ids: List[int] = field(default_factory=list)
    bad_words: List[List[int]] = field(default_factory=list)      # token sequences that may not be produced

    @property
    def has_processors(self) -> bool:
        return bool(self.logit_bias or self.allowed_token_ids or self.bad_words or self.presence_penalty != 0.0
                    or self.frequency_penalty != 0.0 or self.repetition_penalty != 1.0)

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
        if not (-2.0 <= self.presence_penalty <= 2.0):
            raise ValueError("presence_penalty must be in [-2, 2]")
        if not (-2.0 <= self.frequency_penalty <= 2.0):
            raise ValueError("frequency_penalty must be in [-2, 2]")
        if self.repetition_penalty <= 0.0:
            raise ValueError("repetition_penalty must be > 0")
        if self.logprobs > 20:
            raise ValueError("logprobs must be <= 20")
        for t in self.logit_bias:
            if t < 0 or t >= n_vocab:
                raise ValueError(f"logit_bias token id out of range: {t}")
        if self.max_tokens < -1 or self.max_tokens == 0:
            raise ValueError("max_tokens must be >= 1")
        if self.min_tokens < 0:
            raise ValueError("min_tokens must be >= 0")
        if self.max_tokens > 0 and self.min_tokens > self.max_tokens:
            raise ValueError("min_tokens must be <= max_tokens")
        for t in self.stop_token_ids:
            if t < 0 or t >= n_vocab:
                raise ValueError(f"stop_token_ids out of range: {t}")
