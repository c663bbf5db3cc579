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


def row_edits(p: SamplingParams, prompt: Sequence[int], output: Sequence[int], banned: Sequence[int] = ()):
    """What the logits processors do to one row, as ``(allowed ids sorted, {token: [pre, mul_pos, mul_neg, post]})``:
    ``l += pre; l = l * mul_pos if l > 0 else l * mul_neg; l += post``, in the reference's order
    (src/iian/sampler.cpp:72-109): allowed ids, logit bias, bad words, (banned ids while min_tokens holds), penalties.
    """
    edits = {}

    def entry(t):
        return edits.setdefault(int(t), [0.0, 1.0, 1.0, 0.0])

    for t, b in p.logit_bias.items():
        entry(t)[0] += float(b)
    n_out = len(output)
    for bw in p.bad_words:                  # the last token of a sequence whose beginning has just been produced
        if not bw:
            continue
        pre = len(bw) - 1
        if n_out < pre:
            continue
        if all(int(output[n_out - pre + i]) == int(bw[i]) for i in range(pre)):
            entry(bw[-1])[0] = float("-inf")
    for t in banned:
        entry(t)[0] = float("-inf")
    if p.repetition_penalty != 1.0 or p.presence_penalty != 0.0 or p.frequency_penalty != 0.0:
        start = 0 if p.repetition_last_n < 0 else max(0, n_out - p.repetition_last_n)
        counts = {}
        for t in output[start:]:
            counts[int(t)] = counts.get(int(t), 0) + 1
        if p.repetition_penalty != 1.0:     # the repetition penalty applies to prompt tokens as well
            for t in prompt:
                counts.setdefault(int(t), 0)
        for t, c in counts.items():
            e = entry(t)
            if p.repetition_penalty != 1.0:
                e[1], e[2] = 1.0 / p.repetition_penalty, p.repetition_penalty
            if c > 0:
                e[3] -= p.frequency_penalty * c + p.presence_penalty
    return sorted(set(int(t) for t in p.allowed_token_ids)), edits


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device

    def apply_processors(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                         histories: Optional[Sequence] = None, banned: Optional[Sequence[Sequence[int]]] = None) -> None:
        """Run the rows' logits processors on the device: the host only makes the short lists of touched tokens."""
        r, vocab = logits.shape
        allow_off, edit_off, allow_ids, edit_tok = [0], [0], [], []
        vals = [[], [], [], []]
        for row in range(r):
            p = params[row]
            ban = banned[row] if banned is not None else ()
            if p.has_processors or ban:
                prompt, output = histories[row] if histories is not None and p.has_processors else ((), ())
                allowed, edits = row_edits(p, prompt, output, ban)
                allow_ids += [t for t in allowed if 0 <= t < vocab]
                for t, e in edits.items():
                    if 0 <= t < vocab:
                        edit_tok.append(t)
                        for j in range(4):
                            vals[j].append(e[j])
            allow_off.append(len(allow_ids))
            edit_off.append(len(edit_tok))
        if not allow_ids and not edit_tok:
            return
        ints = torch.tensor(allow_off + edit_off + allow_ids + edit_tok, dtype=torch.int32).to(logits.device)
        floats = torch.tensor(vals[0] + vals[1] + vals[2] + vals[3], dtype=torch.float32).to(logits.device)
        ops.kernels().logit_edits(logits, ints, floats, len(allow_ids), len(edit_tok))

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               indices: Sequence[int], banned: Optional[Sequence[Sequence[int]]] = None,
               histories: Optional[Sequence] = None) -> List[int]:
        """One token per logits row.  ``indices[r]`` is the number of tokens request ``r`` has produced
        so far; ``banned[r]`` lists ids that may not be produced now (min_tokens); ``histories[r]`` is the
        request's ``(prompt tokens, output tokens)``, read only for rows whose parameters have processors."""
        r = logits.shape[0]
        if r == 0:
            return []
        k = ops.kernels()
        if banned is not None or any(p.has_processors for p in params):
            self.apply_processors(logits, params, histories, banned)
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

    def logprobs(self, raw_logits: torch.Tensor, tokens: Sequence[int], params: Sequence[SamplingParams]):
        """For every row whose parameters ask for it: ``(log-probability of its token, [(id, log-probability)] of the
        ``logprobs`` most likely tokens)`` under the raw distribution (before any processor); ``None`` for the others."""
        want = [p.logprobs for p in params]
        if all(w < 0 for w in want):
            return [None] * len(want)
        kmax = max(max(want), 0)
        dev = raw_logits.device
        lp, ids, lps = ops.kernels().logprobs(raw_logits, torch.tensor(list(tokens), dtype=torch.int32).to(dev),
                                              torch.tensor(want, dtype=torch.int32).to(dev), kmax)
        lp, ids, lps = lp.tolist(), ids.tolist(), lps.tolist()
        return [None if w < 0 else (lp[r], [(ids[r][j], lps[r][j]) for j in range(min(w, len(ids[r]))) if ids[r][j] >= 0])
                for r, w in enumerate(want)]
