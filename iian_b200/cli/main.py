"""``iian <command>``: complete, bench, random-weights, version.

Commands, option names and meanings follow the reference's command line where it has them
(src/iian/cli/commands.cpp:15-34; ``complete``: src/iian/cli/cmd_run.cpp:225-256; ``bench``:
src/iian/cli/cmd_bench.cpp:18-96; engine, scheduler and sampling flags:
src/iian/cli/engine_options.cpp:26-74).  There is no tokenizer here, so prompts are token ids.
"""
from __future__ import annotations

import json
import random
import sys
import time
from typing import List, Optional

from .args import Options

COMMANDS = ("complete", "bench", "random-weights", "version")


def _add_engine_flags(o: Options) -> None:
    o.group("Engine / KV cache")
    o.add("-c,--max-model-len", "Context length per request, prompt + output (0 = min(model's positions, 8192))", "N", 0, int)
    o.add("--kv-cache-tokens", "Total KV cache capacity in tokens (0 = max-model-len x min(max-num-seqs, 4))", "N", 0, int)
    o.add("--kv-cache-gb", "Cap the KV cache at this many GiB", "G", 0.0, float)
    o.add("--block-size", "KV cache block size in tokens (prefix-cache granularity)", "N", 16, int)
    o.flag("--no-prefix-caching", "Disable automatic prefix caching")
    o.flag("--no-warmup", "Skip the start-up warmup step")
    o.flag("--no-cuda-graphs", "Launch decode steps kernel by kernel instead of replaying captured graphs")
    o.add("--seed", "Base RNG seed for sampling", "N", 0, int)
    o.add("--dtype", "bfloat16 (serving kernels) | float32 (everything in true 32-bit)", "T", "bfloat16", str)
    o.add("--device", "CUDA device index", "N", 0, int)
    o.group("Scheduler")
    o.add("--max-num-seqs", "Max concurrently running requests", "N", 32, int)
    o.add("--max-num-batched-tokens", "Token budget per engine step (chunked-prefill granularity)", "N", 1024, int)
    o.flag("--no-chunked-prefill", "Process prompts whole instead of in chunks")
    o.add("--long-prefill-token-threshold", "Cap a single request's prefill chunk (0 = off)", "N", 0, int)
    o.add("--scheduling-policy", "fcfs | priority", "P", "fcfs", str)
    o.group("Logging")
    o.add("--log-level", "trace|debug|info|warn|error|off", "L", "info", str)
    o.flag("-v,--verbose", "Shortcut for --log-level debug")
    o.flag("-q,--quiet", "Shortcut for --log-level warn")


def _add_sampling_flags(o: Options) -> None:
    o.group("Sampling")
    o.add("-n,--max-tokens", "Max tokens to generate (-1 = until the context is full)", "N", -1, int)
    o.add("--temp", "Temperature (0 = greedy)", "T", 0.7, float)
    o.add("--top-p", "Nucleus sampling", "P", 1.0, float)
    o.add("--top-k", "Top-k sampling (0 = off)", "K", 0, int)
    o.add("--min-p", "Min-p sampling", "P", 0.0, float)
    o.add("--repeat-penalty", "Repetition penalty (1 = off)", "R", 1.0, float)
    o.add("--presence-penalty", "Presence penalty [-2, 2]", "X", 0.0, float)
    o.add("--frequency-penalty", "Frequency penalty [-2, 2]", "X", 0.0, float)
    o.add("--stop", "Stop token ids, e.g. '7,9' (the reference stops on strings; this engine has no tokenizer)", "IDS", "", str)


def engine_config_from_args(ns):
    from ..config.engine import EngineConfig, SchedulerConfig
    return EngineConfig(
        dtype=ns.dtype, max_model_len=ns.max_model_len, kv_cache_tokens=ns.kv_cache_tokens, kv_cache_gb=ns.kv_cache_gb,
        block_size=ns.block_size, enable_prefix_caching=not ns.no_prefix_caching, warmup=not ns.no_warmup,
        seed=ns.seed, cuda_graphs=not ns.no_cuda_graphs, device=ns.device,
        sched=SchedulerConfig(max_num_seqs=ns.max_num_seqs, max_num_batched_tokens=ns.max_num_batched_tokens,
                              enable_chunked_prefill=not ns.no_chunked_prefill,
                              long_prefill_token_threshold=ns.long_prefill_token_threshold, policy=ns.scheduling_policy))


def sampling_from_args(ns):
    from ..sampling.params import SamplingParams
    # one --seed serves as the engine's base seed and, when given, as the request's own seed
    # (src/iian/cli/cmd_run.cpp:37, src/iian/cli/engine_options.cpp:111)
    return SamplingParams(temperature=ns.temp, top_p=ns.top_p, top_k=ns.top_k, min_p=ns.min_p,
                          repetition_penalty=ns.repeat_penalty, presence_penalty=ns.presence_penalty,
                          frequency_penalty=ns.frequency_penalty,
                          stop_token_ids=[int(t) for t in ns.stop.replace(",", " ").split()],
                          seed=ns.seed if "seed" in ns.given else None, max_tokens=ns.max_tokens)


def _log(ns, msg: str) -> None:
    if not ns.quiet and ns.log_level not in ("warn", "error", "off"):
        print(msg, file=sys.stderr, flush=True)


def _parse_ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def cmd_complete(argv: List[str]) -> int:
    o = Options("iian complete", "Completion from token ids (no tokenizer, no chat template).")
    o.positional("model", "model folder (config.json + model.safetensors)")
    o.add("-p,--prompt", "Prompt as token ids, e.g. '1,2,3' ('-' reads them from stdin)", "IDS")
    o.add("--prompt-len", "Instead of -p: a random prompt of this many tokens", "N", 0, int)
    o.add("--prompt-seed", "Seed of the random prompt", "S", 1234, int)
    o.flag("--json", "Print a JSON object with the tokens, their count and the finish reason")
    _add_sampling_flags(o)
    _add_engine_flags(o)
    ns = o.parse(argv)
    from ..engine.engine import Engine
    cfg = engine_config_from_args(ns)
    if "max_num_seqs" not in ns.given:
        cfg.sched.max_num_seqs = 1                      # src/iian/cli/cmd_run.cpp:115
    sp = sampling_from_args(ns)
    if "max_tokens" not in ns.given:
        sp.max_tokens = 128                             # src/iian/cli/cmd_run.cpp:245
    try:
        engine = Engine(ns.model, cfg)
        if ns.prompt:
            prompt = _parse_ids(sys.stdin.read() if ns.prompt == "-" else ns.prompt)
        elif ns.prompt_len > 0:
            rng = random.Random(ns.prompt_seed)
            prompt = [rng.randrange(engine.model.vocab_size) for _ in range(ns.prompt_len)]
        else:
            print("iian complete: missing -p/--prompt (token ids) or --prompt-len", file=sys.stderr)
            return 1
        t0 = time.perf_counter()
        req = engine.submit(prompt, sp)
        while not req.is_finished:
            engine.step()
        secs = time.perf_counter() - t0
    except (ValueError, FileNotFoundError, KeyError, RuntimeError) as e:
        print(f"iian complete: {e}", file=sys.stderr)
        return 1
    toks = req.output_tokens
    if ns.json:
        print(json.dumps({"prompt": prompt, "tokens": toks, "completion_tokens": len(toks),
                          "finish_reason": req.finish_reason.value, "tokens_per_second": len(toks) / secs if secs > 0 else 0.0},
                         indent=2))
    else:
        print(" ".join(str(t) for t in toks))
    return 0


def cmd_bench(argv: List[str]) -> int:
    o = Options("iian bench", "Throughput.  With --concurrency (the reference's form): N concurrent requests with distinct "
                              "random prompts through the scheduler; aggregate tokens/s, time to first token, time per token.  "
                              "With --batch / --prefill-tokens: decode steps and whole-prompt steps timed on the device, with "
                              "the achieved fraction of the HBM and tensor-core rooflines.  With --requests: continuous "
                              "batching of many requests of random lengths, half behind a shared prefix.")
    o.positional("model", "model folder (or leave out and name a --shape with random weights)", nargs="?")
    o.group("Benchmark")
    o.add("--shape", "Random-weight model of a named shape instead of a folder: tinyA | tinyB | 0.6b | 8b | 32b", "NAME", "", str)
    o.add("--layers", "With --shape: run this many layers of the shape (0 = all)", "N", 0, int)
    o.add("--concurrency", "Comma-separated concurrency levels", "LIST", "1,4,16", str)
    o.add("--prompt-tokens", "Prompt length per request", "N", 256, int)
    o.add("--gen-tokens", "Tokens to generate per request (timed decode steps with --batch)", "N", 128, int)
    o.add("--batch", "Comma-separated decode batches, timed on the device with their HBM roofline fraction", "LIST", "", str)
    o.add("--prefill-tokens", "Comma-separated prompt lengths run as one step each, with their tensor-core roofline fraction", "LIST", "", str)
    o.add("--requests", "Continuous batching of this many requests: prompts U[16, 4096], outputs U[16, 512], half sharing "
                        "a 512-token prefix; reports tokens/s, prefix hit rate, preemptions", "N", 0, int)
    o.flag("--json", "Machine-readable output")
    _add_engine_flags(o)
    ns = o.parse(argv)
    from ..engine.engine import Engine
    from ..engine.model import Model
    from ..sampling.params import SamplingParams
    from . import workloads
    if not ns.model and not ns.shape:
        print("iian bench: name a model folder or a --shape", file=sys.stderr)
        return 1
    try:
        if ns.shape:
            model = workloads.random_model(ns.shape, ns.dtype, f"cuda:{ns.device}", layers=ns.layers or None)
        else:
            model = Model.from_folder(ns.model, ns.dtype, f"cuda:{ns.device}")
    except (ValueError, FileNotFoundError, KeyError, RuntimeError) as e:
        print(f"iian bench: {e}", file=sys.stderr)
        return 1
    what = ns.shape or ns.model
    ints = lambda text: [int(x) for x in text.split(",") if x.strip()]
    if ns.requests > 0:
        res = workloads.serving_workload(ns.shape or "model", ns.requests, kv_cache_tokens=ns.kv_cache_tokens,
                                         max_num_seqs=ns.max_num_seqs if "max_num_seqs" in ns.given else 64,
                                         max_num_batched_tokens=ns.max_num_batched_tokens if "max_num_batched_tokens" in ns.given else 2048,
                                         model=model)
        if ns.json:
            print(json.dumps(res, indent=2))
        else:
            print(f"bench {what} | {res['requests']} requests | {res['prompt_tokens']} prompt + {res['generated_tokens']} generated tokens")
            print(f"total {res['total_tok_s']:.0f} tok/s | generation {res['gen_tok_s']:.0f} tok/s | TTFT {res['ttft_ms']:.0f} ms | "
                  f"TPOT {res['tpot_ms']:.1f} ms | prefix hit rate {res['prefix_hit_rate']:.2f} | preemptions {res['preemptions']} | "
                  f"peak cache use {res['kv_usage_peak']:.2f} | wall {res['wall_s']:.1f} s")
        return 0
    if ns.batch or ns.prefill_tokens:
        peaks, kind = workloads.load_peaks()
        res = workloads.decode_and_prefill_points(model, ints(ns.batch), ns.prompt_tokens, ns.gen_tokens, 5, ints(ns.prefill_tokens),
                                                  ns.max_model_len or 8192, peaks, cuda_graphs=not ns.no_cuda_graphs)
        res.pop("engine")
        if ns.json:
            print(json.dumps({"peaks": dict(peaks, kind=kind), "decode": list(res["decode"].values()),
                              "prefill": list(res["prefill"].values())}, indent=2))
            return 0
        print(f"bench {what} | prompt {ns.prompt_tokens} tok | {ns.gen_tokens} timed steps | peaks ({kind}): "
              f"{peaks['hbm_gbs']:.0f} GB/s, {peaks['bf16_tflops']:.0f} TFLOP/s")
        if res["decode"]:
            print(f"{'batch':<8} {'tok/s':>12} {'ms/step':>10} {'GB/s':>10} {'of HBM peak':>12}")
            for b, r in res["decode"].items():
                print(f"{b:<8d} {r['tokens_per_s']:>12.1f} {r['ms_per_step']:>10.3f} {r['hbm_gbs']:>10.0f} {r['roofline_frac']:>12.3f}")
        if res["prefill"]:
            print(f"{'prefill':<8} {'tok/s':>12} {'ms':>10} {'TFLOP/s':>10} {'of bf16 peak':>12}")
            for t, r in res["prefill"].items():
                print(f"{t:<8d} {r['tokens_per_s']:>12.0f} {r['ms']:>10.2f} {r['tflops']:>10.0f} {r['frac']:>12.3f}")
        return 0
    rows = []
    if not ns.json:
        print(f"bench {what} | prompt {ns.prompt_tokens} tok | gen {ns.gen_tokens} tok | dtype {ns.dtype}")
        print(f"{'concurrency':<12} {'prompt tok/s':>14} {'gen tok/s':>14} {'total tok/s':>14} {'TTFT ms':>10} {'TPOT ms':>10} {'wall s':>10}")
    for c in ints(ns.concurrency):
        cfg = engine_config_from_args(ns)
        cfg.sched.max_num_seqs = c                                       # src/iian/cli/cmd_bench.cpp:52-55
        if "max_model_len" not in ns.given:
            cfg.max_model_len = ns.prompt_tokens + ns.gen_tokens + 16
        if "kv_cache_tokens" not in ns.given:
            cfg.kv_cache_tokens = (cfg.max_model_len + cfg.block_size) * c
        cfg.enable_prefix_caching = False
        engine = Engine(model, cfg)
        rng = random.Random(1234)
        sp = SamplingParams(temperature=0.0, max_tokens=ns.gen_tokens, ignore_eos=True)
        v = model.vocab_size
        reqs = [engine.submit([rng.randrange(5, max(6, v - 5)) for _ in range(ns.prompt_tokens)], sp) for _ in range(c)]
        t0 = time.perf_counter()
        while any(not r.is_finished for r in reqs):
            engine.step()
        secs = time.perf_counter() - t0
        st = engine.stats()
        n_gen = sum(r.n_output for r in reqs)
        row = {"concurrency": c, "prompt_tps": c * ns.prompt_tokens / secs, "gen_tps": n_gen / secs,
               "total_tps": (c * ns.prompt_tokens + n_gen) / secs, "ttft_ms": st.ttft_ms_avg, "tpot_ms": st.tpot_ms_avg,
               "wall_s": secs}
        rows.append(row)
        if not ns.json:
            print(f"{c:<12d} {row['prompt_tps']:>14.1f} {row['gen_tps']:>14.1f} {row['total_tps']:>14.1f} "
                  f"{row['ttft_ms']:>10.0f} {row['tpot_ms']:>10.1f} {secs:>10.1f}")
        del engine
    if ns.json:
        print(json.dumps(rows, indent=2))
    return 0


def cmd_random_weights(argv: List[str]) -> int:
    o = Options("iian random-weights", "Write a model folder (config.json, model.safetensors) with random weights "
                                       "from a configuration and a seed.")
    o.positional("model_config", "a config.json (or a folder holding one) that gives the architecture and every size")
    o.positional("out", "folder to write")
    o.add("--seed", "Seed of the weights", "N", 0, int)
    o.add("--std", "Standard deviation of the matrices", "X", 0.02, float)
    o.add("--norm-jitter", "Norm weights are 1 + U(-x, x)", "X", 0.1, float)
    o.add("--store-dtype", "bfloat16 | float32 for the matrices (norm weights are float32)", "T", "bfloat16", str)
    ns = o.parse(argv)
    import os
    import torch
    from ..config.registry import architecture_of
    from ..weights.random_init import write_model_folder
    path = os.path.join(ns.model_config, "config.json") if os.path.isdir(ns.model_config) else ns.model_config
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
        arch = architecture_of(raw)
        cfg = arch.load_config(raw)
        store = {"bfloat16": torch.bfloat16, "float32": torch.float32}[ns.store_dtype]
        write_model_folder(ns.out, arch, cfg, ns.seed, std=ns.std, norm_jitter=ns.norm_jitter, store_dtype=store)
    except (ValueError, FileNotFoundError, KeyError) as e:
        print(f"iian random-weights: {e}", file=sys.stderr)
        return 1
    print(ns.out)
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print("usage: iian <command> [options]\n\ncommands:\n  complete        generate from a prompt of token ids\n"
              "  bench           throughput at several concurrency levels\n  random-weights  write a model folder with random weights\n"
              "  version         print the version\n\n'iian <command> --help' lists a command's options.")
        return 0
    cmd, rest = argv[0], argv[1:]
    if cmd == "version":
        from .. import __version__
        print(f"iian_b200 {__version__}")
        return 0
    if cmd == "complete":
        return cmd_complete(rest)
    if cmd == "bench":
        return cmd_bench(rest)
    if cmd == "random-weights":
        return cmd_random_weights(rest)
    import difflib
    close = difflib.get_close_matches(cmd, COMMANDS, n=1)
    print(f"iian: unknown command '{cmd}'" + (f" (did you mean '{close[0]}'?)" if close else ""), file=sys.stderr)
    return 1


if __name__ == "__main__":
    sys.exit(main())
