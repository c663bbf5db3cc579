"""Sampling next tokens from the step's logits, on the device.

Greedy, temperature, min-p, top-k and top-p follow the reference's CPU sampler
(src/iian/sampler.cpp:111-171; see iian_b200/csrc/sampling.cu for the differences).  The reference
copies every logits row to the host and samples there (src/iian/engine.cpp:606-609, :639-762); here
only token ids cross the bus.

Each request has a stream of uniform numbers of its own: number ``i`` of the stream is a hash of
``(seed, i)``, where ``i`` counts the request's output tokens.  A request's tokens therefore do not
depend on what else is in the batch, on how its prompt was cut, or on being preempted and resumed --
the property the reference gets from a per-request ``mt19937_64`` that advances once per token
(src/iian/sampler.cpp:30-32, :167-168).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import ops
from .params import SamplingParams

_MASK = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15


def _splitmix64(x: int) -> int:
    x = (x + GOLDEN) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform(seed: int, index: int) -> float:
    """Number ``index`` of the stream ``seed``: a float32-exact value in [0, 1)."""
    h = _splitmix64(_splitmix64(seed & _MASK) ^ ((index * 0xD1B54A32D192ED03) & _MASK))
    return (h >> 40) / float(1 << 24)


def request_seed(params: SamplingParams, engine_seed: int, request_id: int) -> int:
    """The request's own seed, or engine seed + id * golden ratio (src/iian/engine.cpp:302)."""
    if params.seed is not None:
        return params.seed & _MASK
    return (engine_seed + request_id * GOLDEN) & _MASK


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               indices: Sequence[int], banned: Optional[Sequence[Sequence[int]]] = None) -> List[int]:
        """One token per logits row.  ``indices[r]`` is the number of tokens request ``r`` has produced
        so far; ``banned[r]`` lists ids that may not be produced now (min_tokens)."""
        r = logits.shape[0]
        if r == 0:
            return []
        k = ops.kernels()
        if banned is not None:
            for row, ids in enumerate(banned):
                if ids:
                    logits[row, torch.as_tensor(list(ids), dtype=torch.long, device=logits.device)] = float("-inf")
        out = torch.empty(r, dtype=torch.int32, device=logits.device)
        if all(p.is_greedy for p in params):
            k.argmax(logits, out)
            return out.tolist()
        host = torch.empty((5, r), dtype=torch.float32)
        for i, p in enumerate(params):
            host[0, i] = p.temperature
            host[1, i] = p.top_p
            host[2, i] = p.min_p
            host[3, i] = uniform(seeds[i], indices[i])
            host[4, i] = float(max(p.top_k, 0))
        dev = host.to(logits.device, non_blocking=False)
        top_k = dev[4].to(torch.int32)
        k.sample(logits, dev[0].contiguous(), top_k, dev[1].contiguous(), dev[2].contiguous(), dev[3].contiguous(), out)
        return out.tolist()
