"""Trace replay: given token ids go through the engine's own model, step function, cache manager and
kernels, step by step; logits come back.  Nothing is sampled and there is no scheduler: the trace is
the schedule.

The reference has no such tool; its nearest piece is a test that builds one batch by hand and reads
the logits of every position (tests/e2e/test-attn-parity.cpp:24-66).

A step is a mapping ``{"step": n, "entries": [{"id", "tokens", "want"}], "end": [ids]}``: each entry
brings a request's next tokens (a request is created by its first entry), ``want`` lists the places
among these tokens whose logits are returned, ``end`` names requests whose pages are given back after
the step.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .model import Model
from .runner import ModelRunner, StepEntry


class TraceError(RuntimeError):
    pass


class TraceReplayer:
    def __init__(self, model: Model, max_tokens: int, block_size: int = 16, max_requests: int = 8, native=None):
        bs = block_size
        self.model = model
        self.max_tokens = max_tokens
        capacity = ((max_tokens + bs - 1) // bs) * bs
        self.runner = ModelRunner(model, block_size=bs, capacity_tokens=capacity, max_num_seqs=max_requests,
                                  enable_prefix_caching=False, native=native)
        self.max_requests = max_requests
        self.live: Dict[object, list] = {}      # id -> [RequestCache, tokens held]

    @classmethod
    def from_folder(cls, model_dir: str, dtype: str, max_tokens: int, block_size: int = 16, max_requests: int = 8,
                    device: str = "cuda:0", native=None) -> "TraceReplayer":
        """``native``: True / False picks the step function in C++ or the one in Python; None takes the default (the
        C++ one for models made of built-in parts)."""
        return cls(Model.from_folder(model_dir, dtype, device), max_tokens, block_size, max_requests, native=native)

    def run_step(self, rec: dict) -> Optional[torch.Tensor]:
        """Run one step; float32 logits ``[wanted, vocab]`` on the device, or None."""
        step = rec.get("step")
        mgr = self.runner.manager
        entries: List[StepEntry] = []
        for ent in rec.get("entries", []):
            rid = ent["id"]
            toks = ent["tokens"]
            if rid not in self.live:
                rc = mgr.new_request()
                if not mgr.allot_state(rc):
                    raise TraceError(f"step {step}: more than {self.max_requests} live requests")
                self.live[rid] = [rc, 0]
            rc, held = self.live[rid]
            for t in toks:
                if not 0 <= int(t) < self.model.vocab_size:
                    raise TraceError(f"step {step}: token id {t} outside the vocabulary ({self.model.vocab_size})")
            if not mgr.allocate(rc, held, len(toks)):
                raise TraceError(f"step {step}: out of cache pages for request {rid!r} ({held} + {len(toks)} tokens; "
                                 f"the cache holds {self.max_tokens})")
            entries.append(StepEntry(rc, toks, held, ent.get("want", [])))
            self.live[rid][1] = held + len(toks)
        logits = self.runner.step(entries) if entries else None
        for rid in rec.get("end", []):
            if rid in self.live:
                mgr.free(self.live[rid][0])
                del self.live[rid]
        return logits
