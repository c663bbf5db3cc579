"""The engine: requests in, tokens out.

Surface and behaviour follow the reference's ``Engine`` (include/iian/engine.h:67-94,
src/iian/engine.cpp): ``submit`` validates and queues a tokenized prompt (engine.cpp:290-326);
``step`` schedules, runs one mixed batch, advances the computed counts, samples one token for every
request whose last token was in the batch, applies the stop rules and frees finished requests
(engine.cpp:456-637, :639-762); ``generate`` submits and steps until everything is finished.
Text, logprobs, grammars, embeddings and speculative decoding are not part of this engine.

Sizing (engine.cpp:105, :131-165): ``max_model_len`` defaults to min(the model's positions, 8192);
the cache holds ``max_model_len * min(max_num_seqs, 4)`` tokens unless told otherwise, capped by
``kv_cache_gb`` or a quarter of the free device memory, and must hold one full-length request.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Union

import torch

from .. import ops
from ..config.engine import EngineConfig
from ..parts.base import KVNeed
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, request_seed
from .model import Model
from .request import FinishReason, OutputChunk, Request, RequestStatus
from .runner import ModelRunner, StepEntry
from .scheduler import Scheduler, SchedulerOutput


@dataclass
class EngineStats:
    requests_total: int = 0
    requests_finished: int = 0
    requests_aborted: int = 0
    prompt_tokens: int = 0
    generation_tokens: int = 0
    cached_prompt_tokens: int = 0
    steps: int = 0
    preemptions: int = 0
    num_running: int = 0
    num_waiting: int = 0
    kv_usage: float = 0.0
    prefix_cache_queries: int = 0
    prefix_cache_hits: int = 0
    ttft_ms_sum: float = 0.0
    ttft_samples: int = 0
    tpot_ms_sum: float = 0.0
    tpot_samples: int = 0

    @property
    def ttft_ms_avg(self) -> float:
        return self.ttft_ms_sum / self.ttft_samples if self.ttft_samples else 0.0

    @property
    def tpot_ms_avg(self) -> float:
        return self.tpot_ms_sum / self.tpot_samples if self.tpot_samples else 0.0


class Engine:
    def __init__(self, model: Union[Model, str], config: Optional[EngineConfig] = None):
        self.cfg = config or EngineConfig()
        self.cfg.validate()
        device = f"cuda:{self.cfg.device}"
        if isinstance(model, str):
            model = Model.from_folder(model, self.cfg.dtype, device)
        self.model = model
        c = self.cfg
        if c.max_model_len > model.max_position:
            raise ValueError(f"max_model_len {c.max_model_len} is beyond the model's {model.max_position} positions "
                             f"(max_position_embeddings)")
        self.max_model_len = c.max_model_len or min(model.max_position, 8192)
        c.sched.max_model_len = self.max_model_len
        bs = c.block_size
        tokens = c.kv_cache_tokens or self.max_model_len * min(c.sched.max_num_seqs, 4)
        per_token = self._cache_bytes_per_token()
        cap_bytes = None
        if c.kv_cache_gb > 0:
            cap_bytes = int(c.kv_cache_gb * (1 << 30))
        elif model.device.type == "cuda" and not c.kv_cache_tokens:
            free, _ = torch.cuda.mem_get_info(model.device)
            cap_bytes = free // 4
        if cap_bytes is not None and per_token > 0:
            tokens = min(tokens, cap_bytes // per_token)
        tokens = (tokens // bs) * bs
        if tokens < self.max_model_len:
            raise ValueError(f"the KV cache holds {tokens} tokens, less than max_model_len {self.max_model_len}; "
                             f"lower --max-model-len or raise --kv-cache-tokens / --kv-cache-gb")
        windows = [n.window for n in model.cache_needs().values() if isinstance(n, KVNeed) and n.window]
        window_cap = None
        if windows:
            window_cap = c.sched.max_num_seqs * (max(windows) + c.sched.max_num_batched_tokens + 2 * bs)
        self.runner = ModelRunner(model, block_size=bs, capacity_tokens=tokens, max_num_seqs=c.sched.max_num_seqs,
                                  enable_prefix_caching=c.enable_prefix_caching, window_capacity_tokens=window_cap,
                                  cuda_graphs=c.cuda_graphs, max_model_len=self.max_model_len)
        self.cache = self.runner.manager
        self.scheduler = Scheduler(c.sched, self.cache)
        self._preemptions_before = 0
        self.sampler = Sampler(model.device)
        self.eos_token_ids = tuple(getattr(model.config, "eos_token_ids", ()) or ())
        self._stats = EngineStats()
        self._requests: Dict[int, Request] = {}
        self._next_id = 1
        self._lock = threading.Lock()
        self._new: List[Request] = []
        self._aborts: List[int] = []
        self._thread: Optional[threading.Thread] = None
        self.logits_hook = None       # optional callable(requests, logits [len(requests), vocab]) run before sampling
        self._quit = False
        self._wake = threading.Condition(self._lock)
        if c.warmup and model.device.type == "cuda":
            self.warmup()

    def _cache_bytes_per_token(self) -> int:
        esize = 2 if self.model.dtype == torch.bfloat16 else 4
        return sum(2 * n.num_kv_heads * n.head_dim * esize for n in self.model.cache_needs().values()
                   if isinstance(n, KVNeed))

    # ---- submission ---------------------------------------------------------------------------
    def submit(self, prompt: Sequence[int], params: Optional[SamplingParams] = None, priority: int = 0,
               cache_salt: int = 0) -> Request:
        params = params or SamplingParams()
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("prompt must not be empty")
        params.validate(self.model.vocab_size)
        for t in prompt:
            if t < 0 or t >= self.model.vocab_size:
                raise ValueError(f"prompt token id out of range: {t}")
        if len(prompt) >= self.max_model_len:
            raise ValueError(f"prompt is too long: {len(prompt)} tokens, max_model_len is {self.max_model_len}")
        with self._wake:
            rid = self._next_id
            self._next_id += 1
            req = Request(id=rid, tokens=prompt, n_prompt=len(prompt), params=params, priority=priority,
                          cache_salt=cache_salt)
            req.seed = request_seed(params, self.cfg.seed, rid)
            self._new.append(req)
            self._requests[rid] = req
            self._stats.requests_total += 1
            self._wake.notify_all()
        return req

    def abort(self, request_id: int) -> None:
        with self._wake:
            self._aborts.append(request_id)
            self._wake.notify_all()

    # ---- one step -----------------------------------------------------------------------------
    def step(self) -> bool:
        """Schedule and run one batch.  False when there was nothing to do."""
        with self._lock:
            fresh, self._new = self._new, []
            aborts, self._aborts = self._aborts, []
        for r in fresh:
            self.scheduler.add_request(r)
        for rid in aborts:
            r = self._requests.get(rid)
            if r is not None and not r.is_finished:
                self._finish(r, RequestStatus.FINISHED_ABORTED, FinishReason.ABORT)
        if not self.scheduler.has_requests:
            return False
        so = self.scheduler.schedule()
        self._stats.preemptions = self.scheduler.num_preemptions - self._preemptions_before
        if not so.scheduled:
            if so.preempted:
                return True
            if not self.scheduler.running:
                for r in list(self.scheduler.waiting):     # cannot fit even alone (engine.cpp:477-485)
                    self._finish(r, RequestStatus.FINISHED_ERROR, FinishReason.ERROR,
                                 "request does not fit in the KV cache")
            return False

        entries: List[StepEntry] = []
        sampled: List[Request] = []
        for s in so.scheduled:
            r = s.req
            start = r.num_computed_tokens
            reaches_end = start + s.n_new_tokens >= r.n_tokens
            entries.append(StepEntry(r.cache, r.tokens[start:start + s.n_new_tokens], start,
                                     [s.n_new_tokens - 1] if reaches_end else []))
            if reaches_end:
                sampled.append(r)
        logits = self.runner.step(entries)
        self._stats.steps += 1
        n_prompt_done = 0
        for s in so.scheduled:
            before = s.req.num_computed_tokens
            if before < s.req.n_prompt:
                n_prompt_done += min(s.n_new_tokens, s.req.n_prompt - before)
        self.scheduler.update_after_step(so)
        self._stats.prompt_tokens += n_prompt_done
        if sampled:
            if self.logits_hook is not None:
                self.logits_hook(sampled, logits)
            self._process_outputs(sampled, logits)
        return True

    def _process_outputs(self, reqs: List[Request], logits: torch.Tensor) -> None:
        banned = None
        if any(r.n_output < r.params.min_tokens for r in reqs):
            banned = [list(self.eos_token_ids) + list(r.params.stop_token_ids) if r.n_output < r.params.min_tokens else []
                      for r in reqs]
        histories = None
        if any(r.params.has_processors for r in reqs):      # (prompt, output) of the rows whose processors read them
            histories = [(r.tokens[:r.n_prompt], r.tokens[r.n_prompt:]) if r.params.has_processors else ((), ())
                         for r in reqs]
        want_lp = any(r.params.logprobs >= 0 for r in reqs)
        raw = logits.clone() if want_lp and (banned is not None or histories is not None) else logits
        tokens = self.sampler.sample(logits, [r.params for r in reqs], [r.seed for r in reqs],
                                     [r.n_output for r in reqs], banned, histories)
        if want_lp:                                       # of the raw distribution, as the reference reports them
            for r, lp in zip(reqs, self.sampler.logprobs(raw, tokens, [r.params for r in reqs])):
                if lp is not None:
                    r.pending_logprobs.append(lp)
                    r.logprobs.append(lp)
        self.runner.check_device_status()      # the tokens are on the host: a kernel that gave up has said so by now
        now = time.monotonic()
        for r, tok in zip(reqs, tokens):
            r.tokens.append(tok)
            r.pending_tokens.append(tok)
            self._stats.generation_tokens += 1
            if r.n_output == 1:
                r.t_first_token = now
                self._stats.ttft_ms_sum += (now - r.arrival) * 1e3
                self._stats.ttft_samples += 1
            else:
                self._stats.tpot_ms_sum += (now - r.t_last_token) * 1e3
                self._stats.tpot_samples += 1
            r.t_last_token = now
            p = r.params
            stop, why = False, FinishReason.NONE
            if tok in self.eos_token_ids and not p.ignore_eos:
                stop, why = True, FinishReason.STOP
            if not stop and tok in p.stop_token_ids:
                stop, why = True, FinishReason.STOP
                r.stop_reason = str(tok)
            if not stop and p.max_tokens > 0 and r.n_output >= p.max_tokens:
                stop, why = True, FinishReason.LENGTH
            if not stop and r.n_tokens >= self.max_model_len:
                stop, why = True, FinishReason.LENGTH
            if stop:
                self._finish(r, RequestStatus.FINISHED_LENGTH if why == FinishReason.LENGTH
                             else RequestStatus.FINISHED_STOPPED, why)
            else:
                self._deliver(r, False)

    def _deliver(self, r: Request, final: bool) -> None:
        chunk = OutputChunk(tokens=r.pending_tokens, logprobs=r.pending_logprobs, finished=final,
                            finish_reason=r.finish_reason, stop_reason=r.stop_reason, error=r.error,
                            n_prompt_tokens=r.n_prompt, n_output_tokens=r.n_output, n_cached_tokens=r.num_cached_tokens)
        r.pending_tokens = []
        r.pending_logprobs = []
        r.outputs.append(chunk)

    def _finish(self, r: Request, status: RequestStatus, why: FinishReason, error: str = "") -> None:
        r.finish_reason = why
        r.error = error
        r.t_finished = time.monotonic()
        self.scheduler.finish_request(r, status)
        self._stats.requests_finished += 1
        if why == FinishReason.ABORT:
            self._stats.requests_aborted += 1
        self._stats.cached_prompt_tokens += r.num_cached_tokens
        self._deliver(r, True)
        self._requests.pop(r.id, None)

    # ---- conveniences -------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 max_tokens: Optional[int] = None, temperature: Optional[float] = None, seed: Optional[int] = None
                 ) -> List[List[int]]:
        """Generated token ids for each prompt (host lists in, host lists out)."""
        if params is None or isinstance(params, SamplingParams):
            base = params or SamplingParams(temperature=0.0)
            plist = []
            for i in range(len(prompts)):
                p = SamplingParams(**{**base.__dict__})
                if max_tokens is not None:
                    p.max_tokens = max_tokens
                if temperature is not None:
                    p.temperature = temperature
                if seed is not None:
                    p.seed = seed + i
                plist.append(p)
        else:
            plist = list(params)
        reqs = [self.submit(pr, p) for pr, p in zip(prompts, plist)]
        while any(not r.is_finished for r in reqs):
            if not self.step() and any(not r.is_finished for r in reqs) and not self.scheduler.has_requests \
                    and not self._new:
                break
        for r in reqs:
            if r.finish_reason == FinishReason.ERROR:
                raise RuntimeError(f"request {r.id}: {r.error}")
        return [r.output_tokens for r in reqs]

    def warmup(self) -> None:
        """A small prefill and two decode steps, so that kernels are compiled and loaded before the
        first request (src/iian/engine.cpp:252-276)."""
        n = max(1, min(64, self.max_model_len - 4, self.cfg.sched.max_num_batched_tokens))
        saved = self._stats
        try:
            r = self.submit([0] * n, SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True), cache_salt=0x7761726D)
            while not r.is_finished:
                if not self.step():
                    break
        finally:
            self._stats = EngineStats()
            self._next_id = 1
            for pool in self.cache.pools:
                pool.reset_prefix_cache()
            self._preemptions_before = self.scheduler.num_preemptions      # the warm-up's do not count
            del saved

    def stats(self) -> EngineStats:
        s = self._stats
        s.num_running = len(self.scheduler.running)
        s.num_waiting = len(self.scheduler.waiting)
        s.kv_usage = self.cache.usage
        s.prefix_cache_queries = self.cache.prefix_queries
        s.prefix_cache_hits = self.cache.prefix_hits
        s.preemptions = self.scheduler.num_preemptions - self._preemptions_before
        return s

    # ---- background loop (include/iian/engine.h:71-72) ------------------------------------------
    def start(self) -> None:
        if self._thread is not None:
            return
        self._quit = False
        self._thread = threading.Thread(target=self._run_loop, name="iian-engine", daemon=True)
        self._thread.start()

    def _run_loop(self) -> None:
        if self.model.device.type == "cuda":
            torch.cuda.set_device(self.model.device)
        while True:
            with self._wake:
                while not self._quit and not self._new and not self._aborts and not self.scheduler.has_requests:
                    self._wake.wait(0.05)
                if self._quit:
                    return
            try:
                self.step()
            except Exception as e:  # a failed step ends every request with an error (engine.cpp:391-396)
                for r in self.scheduler.all_requests():
                    self._finish(r, RequestStatus.FINISHED_ERROR, FinishReason.ERROR, str(e))

    def stop(self) -> None:
        with self._wake:
            self._quit = True
            self._wake.notify_all()
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        for r in self.scheduler.all_requests():
            self._finish(r, RequestStatus.FINISHED_ABORTED, FinishReason.ABORT, "engine shutting down")
