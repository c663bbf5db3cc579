"""The benchmark workloads: model shapes by name, device-timed decode and prefill with their rooflines, and
continuous batching of many requests through the scheduler.

``iian bench --shape ...`` and the repository's ``bench.py`` both call this module.  The method is the
reference's (tests/e2e/bench-batch.cpp:45-84, src/iian/cli/cmd_bench.cpp:18-96): random weights, seeded uniform
random token ids, greedy, ``ignore_eos``; wall clock for the scheduler-driven runs (TTFT = time to a request's
first token, TPOT = mean time between its tokens), CUDA events around the step function for the device-timed
figures.  Rooflines: a decode step has to read every weight it uses once and the cache of its live requests
(HBM bytes / time against the measured copy bandwidth); a prefill step's flops / time against the measured
bfloat16 matrix-product peak.
"""
from __future__ import annotations

import json
import os
import random
import statistics
import time
from typing import Dict, List, Optional, Sequence

# name -> config.json keys of the shape (random weights; no checkpoint is read)
SHAPES: Dict[str, dict] = {
    "tinyA": dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, rope_theta=10000.0,
                  max_position_embeddings=128, tie_word_embeddings=True),
    "tinyB": dict(vocab_size=503, hidden_size=96, intermediate_size=160, num_hidden_layers=3, num_attention_heads=8,
                  num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-5, rope_theta=1000000.0,
                  max_position_embeddings=256, tie_word_embeddings=False),
    "0.6b": dict(vocab_size=151936, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
                 num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
                 max_position_embeddings=40960, tie_word_embeddings=True),
    "8b": dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
               max_position_embeddings=40960, tie_word_embeddings=False),
    "32b": dict(vocab_size=151936, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64,
                num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
                max_position_embeddings=40960, tie_word_embeddings=False),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks(root: Optional[str] = None):
    """Measured copy bandwidth and bfloat16 product peak of this pool's GPUs if ``MEASURED_PEAKS.json`` lies in
    ``root`` (the repository), else the stated fallback: ``(peaks, "measured" | "fallback")``."""
    root = root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                    "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"]))}, "measured"
        except (KeyError, ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def shape_config(name: str, layers: Optional[int] = None):
    from ..models.qwen3 import qwen3_config_from_dict
    try:
        raw = dict(SHAPES[name])
    except KeyError:
        raise ValueError(f"unknown shape '{name}' ({' | '.join(SHAPES)})") from None
    if layers:
        raw["num_hidden_layers"] = layers
    return qwen3_config_from_dict(raw)


def random_model(name: str, dtype: str = "bfloat16", device="cuda:0", seed: int = 0, layers: Optional[int] = None):
    """The shape ``name`` with random weights N(0, 0.02) and norm weights 1, drawn on the device."""
    from ..config.registry import get_architecture
    from ..engine.model import Model
    cfg = shape_config(name, layers)
    return Model.from_random(get_architecture("Qwen3ForCausalLM"), cfg, seed=seed, dtype=dtype, device=device, norm_jitter=0.0)


class Accounting:
    """Bytes and flops of a dense Qwen3 step, from the configuration."""

    def __init__(self, cfg, dtype_bytes: int = 2):
        self.cfg = cfg
        self.layer_w = cfg.hidden_size * (cfg.q_size + 2 * cfg.kv_size) + cfg.q_size * cfg.hidden_size \
            + 3 * cfg.hidden_size * cfg.intermediate_size
        self.head_w = cfg.vocab_size * cfg.hidden_size
        self.weight_bytes_step = dtype_bytes * (cfg.num_hidden_layers * self.layer_w + self.head_w)
        self.kv_bytes_token = cfg.num_hidden_layers * 2 * cfg.kv_size * dtype_bytes

    def decode_bytes(self, batch: int, ctx_avg: float) -> float:
        return self.weight_bytes_step + batch * ctx_avg * self.kv_bytes_token

    def prefill_flops(self, tokens: int) -> float:
        c = self.cfg
        return 2.0 * tokens * c.num_hidden_layers * self.layer_w + 2.0 * self.head_w \
            + c.num_hidden_layers * 4.0 * c.q_size * tokens * (tokens + 1) / 2


class TokenSource:
    def __init__(self, vocab: int, seed: int = 1234):
        import torch
        self.vocab = vocab
        self.gen = torch.Generator().manual_seed(seed)

    def take(self, n: int) -> List[int]:
        import torch
        return torch.randint(5, max(6, self.vocab - 5), (n,), generator=self.gen).tolist()


def prefill_requests(runner, source: TokenSource, batch: int, prompt_len: int, budget: int = 2048):
    """``batch`` requests with ``prompt_len`` random tokens each in the cache (several prompts to a step)."""
    from ..engine.runner import StepEntry
    mgr = runner.manager
    caches = []
    for _ in range(batch):
        rc = mgr.new_request()
        mgr.allot_state(rc)
        caches.append(rc)
    per_step = max(1, budget // prompt_len)
    for i in range(0, batch, per_step):
        ents = []
        for rc in caches[i:i + per_step]:
            if not mgr.allocate(rc, 0, prompt_len):
                raise RuntimeError("the cache is too small for this batch of prompts")
            ents.append(StepEntry(rc, source.take(prompt_len), 0, []))
        runner.step(ents)
    return caches


def measure_decode(runner, source: TokenSource, batch: int, prompt_len: int, warmup: int, steps: int) -> dict:
    """Decode ``batch`` requests from prompts of ``prompt_len`` tokens: ``warmup`` untimed steps, then ``steps`` steps of
    the step function plus the on-device argmax between two CUDA events.  Each step streams every weight from HBM
    (they exceed the L2 many times), so nothing survives in the L2 between timed iterations."""
    import torch
    from .. import ops
    from ..engine.runner import StepEntry
    kern, mgr, dev = ops.kernels(), runner.manager, runner.device
    caches = prefill_requests(runner, source, batch, prompt_len)
    out = torch.empty(batch, dtype=torch.int32, device=dev)
    toks = source.take(batch)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pos, launches0 = prompt_len, 0
    for i in range(warmup + steps):
        if i == warmup:
            torch.cuda.synchronize()
            launches0 = runner.launches
            start.record()
        ents = []
        for rc, t in zip(caches, toks):
            if not mgr.allocate(rc, pos, 1):
                raise RuntimeError("out of cache pages while decoding")
            ents.append(StepEntry(rc, [t], pos, [0]))
        logits = runner.step(ents)
        kern.argmax(logits, out)
        pos += 1
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    launches = runner.launches - launches0 + steps
    for rc in caches:
        mgr.free(rc)
    return {"batch": batch, "ms_per_step": ms, "tokens_per_s": batch / (ms * 1e-3), "launches": int(launches),
            "ctx_avg": prompt_len + warmup + (steps + 1) / 2}


def measure_prefill(runner, source: TokenSource, tokens: int, warmup: int = 3, repeats: int = 5) -> dict:
    """One prompt of ``tokens`` tokens as one step; the median of ``repeats`` runs after ``warmup`` runs."""
    import torch
    from ..engine.runner import StepEntry
    mgr = runner.manager
    toks = source.take(tokens)
    times = []
    for i in range(warmup + repeats):
        rc = mgr.new_request()
        mgr.allot_state(rc)
        if not mgr.allocate(rc, 0, tokens):
            raise RuntimeError("the cache is too small for this prompt")
        s_ev, e_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s_ev.record()
        runner.step([StepEntry(rc, toks, 0, [tokens - 1])])
        e_ev.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(s_ev.elapsed_time(e_ev))
        mgr.free(rc)
    ms = statistics.median(times)
    return {"tokens": tokens, "ms": ms, "tokens_per_s": tokens / (ms * 1e-3)}


def decode_and_prefill_points(model, batches: Sequence[int], prompt_len: int, steps: int, warmup: int,
                              prefill_tokens: Sequence[int], context_len: int, peaks: dict, cuda_graphs: bool = True) -> dict:
    """Decode at every batch of ``batches`` and prefill at every length of ``prefill_tokens`` for one model, with the
    roofline fractions: ``{"decode": {B: {...}}, "prefill": {T: {...}}}``."""
    from ..config.engine import EngineConfig, SchedulerConfig
    from ..engine.engine import Engine
    acc = Accounting(model.config)
    max_b = max(batches) if batches else 1
    per_req = prompt_len + warmup + steps + 48
    longest = max([per_req] + list(prefill_tokens))
    max_len = -(-max(context_len, longest + 16) // 16) * 16       # whole pages
    ecfg = EngineConfig(dtype="bfloat16", max_model_len=max_len, kv_cache_tokens=max(max_len, max_b * per_req),
                        block_size=16, enable_prefix_caching=False, warmup=True, cuda_graphs=cuda_graphs,
                        sched=SchedulerConfig(max_num_seqs=max(1, max_b), max_num_batched_tokens=max(2048, longest)))
    engine = Engine(model, ecfg)
    src = TokenSource(model.vocab_size)
    out = {"decode": {}, "prefill": {}, "engine": engine}
    for b in batches:
        r = measure_decode(engine.runner, src, b, prompt_len, warmup, steps)
        nbytes = acc.decode_bytes(b, r["ctx_avg"])
        r["hbm_gbs"] = nbytes / (r["ms_per_step"] * 1e-3) / 1e9
        r["roofline_frac"] = r["hbm_gbs"] / peaks["hbm_gbs"]
        r["bytes_per_step"] = nbytes
        out["decode"][b] = r
    for t in prefill_tokens:
        r = measure_prefill(engine.runner, src, t, warmup=max(2, min(warmup, 3)))
        flops = acc.prefill_flops(t)
        r["tflops"] = flops / (r["ms"] * 1e-3) / 1e12
        r["frac"] = r["tflops"] / peaks["bf16_tflops"]
        out["prefill"][t] = r
    return out


# ---- continuous batching of many requests (BASELINE's Qwen3-0.6B workload) -----------------------------------
def serving_requests(vocab: int, n_requests: int, prompt_range=(16, 4096), output_range=(16, 512), shared_prefix: int = 512,
                     shared_fraction: float = 0.5, seed: int = 7):
    """``n_requests`` (prompt, output length) pairs: prompt lengths uniform in ``prompt_range``, output lengths
    uniform in ``output_range``, uniform random token ids; ``shared_fraction`` of the requests begin with the same
    ``shared_prefix`` tokens (their length is then at least that prefix plus one token)."""
    rng = random.Random(seed)
    prefix = [rng.randrange(5, max(6, vocab - 5)) for _ in range(shared_prefix)]
    out = []
    for i in range(n_requests):
        n = rng.randint(*prompt_range)
        n_out = rng.randint(*output_range)
        shares = rng.random() < shared_fraction
        if shares:
            n = max(n, shared_prefix + 1)
            toks = prefix + [rng.randrange(5, max(6, vocab - 5)) for _ in range(n - shared_prefix)]
        else:
            toks = [rng.randrange(5, max(6, vocab - 5)) for _ in range(n)]
        out.append((toks, n_out, shares))
    return out


def run_serving(engine, requests, check_alone: int = 0) -> dict:
    """Submit every request at once, step until all are finished (wall clock), and report throughput, latencies,
    prefix-cache hit rate, preemptions and the peak cache usage.  ``check_alone``: afterwards (untimed) that many of
    the requests are run again one at a time and their greedy tokens compared with what they produced in the crowd
    (``alone_mismatches`` counts requests whose tokens differ before their first near-tie cannot be told: in
    bfloat16 a different batch changes the rounding, so only the agreeing prefix length is reported)."""
    import torch
    from ..sampling.params import SamplingParams
    reqs = []
    for toks, n_out, _ in requests:
        reqs.append(engine.submit(toks, SamplingParams(temperature=0.0, max_tokens=n_out, ignore_eos=True)))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    peak_usage, steps = 0.0, 0
    while engine.step():               # False once no request is left to run
        steps += 1
        if steps % 8 == 0:
            peak_usage = max(peak_usage, engine.cache.usage)
    torch.cuda.synchronize()
    secs = time.perf_counter() - t0
    st = engine.stats()
    n_prompt = sum(len(t) for t, _, _ in requests)
    n_gen = sum(r.n_output for r in reqs)
    errors = sum(1 for r in reqs if not r.is_finished or r.finish_reason.value == "error")
    out = {"requests": len(reqs), "wall_s": secs, "steps": steps, "prompt_tokens": n_prompt, "generated_tokens": n_gen,
           "total_tok_s": (n_prompt + n_gen) / secs, "gen_tok_s": n_gen / secs, "prompt_tok_s": n_prompt / secs,
           "ttft_ms": st.ttft_ms_avg, "tpot_ms": st.tpot_ms_avg,
           "prefix_queries": st.prefix_cache_queries, "prefix_hits": st.prefix_cache_hits,
           "prefix_hit_rate": st.prefix_cache_hits / st.prefix_cache_queries if st.prefix_cache_queries else 0.0,
           "cached_prompt_tokens": st.cached_prompt_tokens, "preemptions": st.preemptions, "kv_usage_peak": peak_usage,
           "errors": errors}
    if check_alone:
        step = max(1, len(reqs) // check_alone)
        agree, total, full = 0, 0, 0
        for i in list(range(0, len(reqs), step))[:check_alone]:
            toks, n_out, _ = requests[i]
            n_cmp = min(n_out, 32)
            r = engine.submit(toks, SamplingParams(temperature=0.0, max_tokens=n_cmp, ignore_eos=True))
            while not r.is_finished:
                engine.step()
            a, b = r.output_tokens, reqs[i].output_tokens[:n_cmp]
            k = 0
            while k < len(a) and k < len(b) and a[k] == b[k]:
                k += 1
            agree += k
            total += n_cmp
            full += int(k == n_cmp)
        out["alone_checked"] = check_alone
        out["alone_identical"] = full
        out["alone_agreeing_token_share"] = agree / total if total else 1.0
    return out


def serving_workload(shape: str = "0.6b", n_requests: int = 256, kv_cache_tokens: int = 0, max_num_seqs: int = 64,
                     max_num_batched_tokens: int = 2048, seed: int = 7, check_alone: int = 8, device="cuda:0",
                     prompt_range=(16, 4096), output_range=(16, 512), shared_prefix: int = 512, model=None) -> dict:
    """BASELINE's continuous-batching workload: ``n_requests`` requests, prompts U[16, 4096], outputs U[16, 512],
    half sharing a 512-token prefix, through the scheduler with prefix reuse on and a cache small enough that
    requests are preempted (by default a third of what the running requests could hold at their longest)."""
    from ..config.engine import EngineConfig, SchedulerConfig
    from ..engine.engine import Engine
    model = model or random_model(shape, "bfloat16", device)
    max_len = prompt_range[1] + output_range[1] + 16
    if not kv_cache_tokens:
        kv_cache_tokens = max(max_len, max_num_seqs * max_len // 3)
    ecfg = EngineConfig(dtype="bfloat16", max_model_len=max_len, kv_cache_tokens=kv_cache_tokens, block_size=16,
                        enable_prefix_caching=True, warmup=True, cuda_graphs=True,
                        sched=SchedulerConfig(max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens))
    engine = Engine(model, ecfg)
    reqs = serving_requests(model.vocab_size, n_requests, prompt_range, output_range, shared_prefix, 0.5, seed)
    out = run_serving(engine, reqs, check_alone)
    out.update({"shape": shape, "kv_cache_tokens": kv_cache_tokens, "max_num_seqs": max_num_seqs,
                "max_num_batched_tokens": max_num_batched_tokens})
    return out
