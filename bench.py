#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the Qwen3-8B layer sizes, random weights, one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

A "step" is one decode step of a batch.  ``value`` is decoded tokens per second measured on the
device (CUDA events around K steps of the step function plus the on-device argmax); ``e2e`` is the
same through the Python entry point (``Engine.step``: scheduler, upload of the step's integers from
pinned memory, model, sampling, token ids back to the host).  ``prefill`` is one 2,048-token prompt;
``roofline`` compares the bytes a decode step has to read (every weight once, the cache of the live
requests) with the measured HBM copy bandwidth; ``points`` gives decode at batch 1 and 64.

Inputs are larger than L2: a decode step streams 15 GB of weights, a prefill step 14 GB, so nothing
survives in the 126 MB L2 between timed iterations.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from iian_b200.cli.workloads import SHAPES  # noqa: E402  (shapes by name; no CUDA is touched by the import)

SHAPE_8B = SHAPES["8b"]     # BASELINE.json configs[2]
CONTEXT_LEN = 8192          # the engine's max_model_len for the benchmark
PROMPT_LEN = 1024           # decode starts from prompts of this many random tokens
PREFILL_TOKENS = 2048


def reference_arm(args) -> int:
    """``--impl reference``: the unmodified reference (built with CMake under ``baseline/_ref``) through its own
    command line, ``iian bench <gguf> --concurrency B --prompt-tokens 1024 --gen-tokens N --json``, on the same shape
    with the same random weights, written as a bfloat16 GGUF into a temporary folder.  Nothing of this repository's
    engine is on that path.  ``value`` is its decode rate, B / TPOT (its own mean time between a request's tokens);
    the same figure stands as ``e2e``, because the reference's bench is end to end by construction (token ids from
    the host through its public Engine API, tokens and text back)."""
    import shutil
    import tempfile
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ra
    why = ra.available()
    if why is None and args.gpus != 1:
        why = "the reference's bench runs on one GPU"
    if why is not None:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    K, W, B = args.steps, max(3, args.warmup), args.batch
    shape = dict(SHAPE_8B, num_hidden_layers=args.layers)
    work = tempfile.mkdtemp(prefix="iian_ref_")
    try:
        import torch
        t0 = time.time()
        path = os.path.join(work, "model.gguf")
        nbytes = ra.write_gguf(path, shape, seed=0, device="cuda:0" if torch.cuda.is_available() else "cpu")
        print(f"[bench] reference model written in {time.time() - t0:.1f} s ({nbytes / 1e9:.2f} GB)", file=sys.stderr)
        torch.cuda.empty_cache()
        sampler = ClockSampler(0)
        sampler.start()
        try:
            row = ra.run_bench(path, B, PROMPT_LEN, W + K, extra=["--block-size", "16"])
        finally:
            sampler.stop()
    except Exception as e:  # noqa: BLE001  (whatever went wrong, the arm says so in one line and the run goes on)
        print(json.dumps({"impl": "reference", "unavailable": f"the reference did not run: {str(e)[:300]}"}))
        return 0
    finally:
        shutil.rmtree(work, ignore_errors=True)
    decode_tps = B * 1000.0 / row["tpot_ms"] if row.get("tpot_ms") else 0.0
    line = {
        "impl": "reference",
        "metric": "decode tokens/s (Qwen3-8B shape, batch 8)" if B == 8 else f"decode tokens/s (Qwen3-8B shape, batch {B})",
        "value": decode_tps, "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": row.get("tpot_ms"),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02) (the same values as the other arm), uniform random token ids (the reference's own)",
        "config": {"model": "Qwen3-8B shape (BASELINE.json configs[2])", "global_batch": B, "seq_len": PROMPT_LEN,
                   "parallelism": "single GPU", "layers": shape["num_hidden_layers"], "layers_of_config": SHAPE_8B["num_hidden_layers"],
                   "hidden": shape["hidden_size"], "heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
                   "head_dim": shape["head_dim"], "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
                   "context_len": PROMPT_LEN + W + K + 16, "prompt_len": PROMPT_LEN, "kv_block": 16,
                   "command": "iian bench --concurrency B --prompt-tokens 1024 --gen-tokens W+K --json", "kv_dtype": "f16 (its default)"},
        "e2e": {"value": decode_tps, "unit": "tokens/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                "ms_per_step": row.get("tpot_ms")},
        "clocks": sampler.summary(),
        "reference_row": {k: row[k] for k in ("concurrency", "prompt_tps", "gen_tps", "total_tps", "ttft_ms", "tpot_ms", "wall_s") if k in row},
    }
    print(json.dumps(line))
    return 0


class ClockSampler:
    """nvidia-smi in a loop while a timed region runs; reads only."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device = device
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.rows.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm = [int(r[0]) for r in self.rows if r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=SHAPE_8B["num_hidden_layers"],
                    help="run fewer layers than the configuration has (reported in config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cuda-graphs", action="store_true")
    ap.add_argument("--skip-points", action="store_true", help="the headline and the end-to-end figure only")
    ap.add_argument("--skip-32b", action="store_true", help="leave out the Qwen3-32B shape")
    ap.add_argument("--skip-serve", action="store_true", help="leave out the continuous-batching workload (Qwen3-0.6B shape)")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    K, W = args.steps, max(3, args.warmup)

    import gc
    import torch
    from iian_b200 import EngineConfig, SamplingParams, SchedulerConfig
    from iian_b200 import ops
    from iian_b200.cli import workloads as wl
    from iian_b200.engine.engine import Engine
    from iian_b200.engine.runner import StepEntry

    peaks, peak_kind = wl.load_peaks(ROOT)
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    t_build = time.time()
    model = wl.random_model("8b", "bfloat16", dev, seed=0, layers=args.layers)
    cfg = model.config
    acc = wl.Accounting(cfg)
    max_b = max(args.batch, 1 if args.skip_points else 64)
    per_req = PROMPT_LEN + W + K + 48
    longest_prefill = PREFILL_TOKENS if args.skip_points else max(PREFILL_TOKENS, 8192)
    long_ctx = 0 if args.skip_points else 8192 + W + K + 64          # the decode points at 8,192 tokens of context
    ecfg = EngineConfig(dtype="bfloat16", max_model_len=max(CONTEXT_LEN, longest_prefill + 64, long_ctx),
                        kv_cache_tokens=max(CONTEXT_LEN, longest_prefill + 64, max_b * per_req, 8 * long_ctx),
                        block_size=16, enable_prefix_caching=False, warmup=True, cuda_graphs=not args.no_cuda_graphs,
                        sched=SchedulerConfig(max_num_seqs=max_b, max_num_batched_tokens=2048))
    engine = Engine(model, ecfg)
    runner, kern = engine.runner, ops.kernels()
    print(f"[bench] model and engine ready in {time.time() - t_build:.1f} s "
          f"({model.weight_bytes / 1e9:.2f} GB of weights, cache {runner.storage.bytes / 1e9:.2f} GB)", file=sys.stderr)
    src = wl.TokenSource(cfg.vocab_size, 1234)

    # ---- timed: decode at the headline batch (device clock) -------------------------------------
    sampler = ClockSampler(0)
    sampler.start()
    B = args.batch
    head = wl.measure_decode(runner, src, B, PROMPT_LEN, W, K)
    ms_step, launches, ctx_avg = head["ms_per_step"], head["launches"], head["ctx_avg"]
    value = head["tokens_per_s"]
    bytes_step = acc.decode_bytes(B, ctx_avg)
    achieved = bytes_step / (ms_step * 1e-3) / 1e9

    # ---- timed: the same through the Python entry point (host tokens in and out) -----------------
    sp = SamplingParams(temperature=0.0, max_tokens=W + K + 8, ignore_eos=True)
    reqs = [engine.submit(src.take(PROMPT_LEN), sp) for _ in range(B)]
    while any(r.n_output < W for r in reqs):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n0 = sum(r.n_output for r in reqs)
    for _ in range(K):
        engine.step()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    e2e_tokens = sum(r.n_output for r in reqs) - n0
    e2e = {"value": e2e_tokens / (t1 - t0), "unit": "tokens/s", "h2d_bytes_per_step": int(runner.last_upload_bytes),
           "d2h_bytes_per_step": 4 * B, "ms_per_step": (t1 - t0) * 1e3 / K}
    for r in reqs:
        engine.abort(r.id)
    engine.step()

    points, prefill, check = {}, None, None
    if not args.skip_points:
        for b in (1, 64):
            r = wl.measure_decode(runner, src, b, PROMPT_LEN, W, K)
            points[f"decode_b{b}"] = r["tokens_per_s"]
            points[f"decode_b{b}_hbm_frac"] = acc.decode_bytes(b, r["ctx_avg"]) / (r["ms_per_step"] * 1e-3) / 1e9 / peaks["hbm_gbs"]
        # ---- decode at a context of 8,192 tokens (attention reads eight times the K/V of the headline's) ----------
        for b in (1, 8):
            r = wl.measure_decode(runner, src, b, 8192, W, max(8, K // 2))
            points[f"decode_b{b}_ctx8k"] = r["tokens_per_s"]
            points[f"decode_b{b}_ctx8k_hbm_frac"] = acc.decode_bytes(b, r["ctx_avg"]) / (r["ms_per_step"] * 1e-3) / 1e9 / peaks["hbm_gbs"]
        # ---- prefill of one 2,048-token prompt (and of 512 and 8,192 tokens) ---------------------------
        for T in (PREFILL_TOKENS, 512, 8192):
            r = wl.measure_prefill(runner, src, T, warmup=W if T == PREFILL_TOKENS else 2, repeats=5 if T == PREFILL_TOKENS else 3)
            flops = acc.prefill_flops(T)
            if T == PREFILL_TOKENS:
                prefill = {"value": r["tokens_per_s"], "tokens": T, "ms": r["ms"],
                           "frac": flops / (r["ms"] * 1e-3) / (peaks["bf16_tflops"] * 1e12), "tflops": flops / (r["ms"] * 1e-3) / 1e12}
            else:
                points[f"prefill_{T}"] = r["tokens_per_s"]
                points[f"prefill_{T}_frac"] = flops / (r["ms"] * 1e-3) / (peaks["bf16_tflops"] * 1e12)
    sampler.stop()
    if hasattr(kern, "tcgen05_check"):
        kern.tcgen05_check(dev)          # a tcgen05 kernel that gave up on a barrier would have left garbage

    if not args.skip_points:
        # ---- untimed: the bfloat16 path against the true 32-bit path on a 2-layer cut of the same model ------
        # (the generator is keyed by tensor name, so the cut has the full model's embedding, first layers and head)
        del engine, runner, model
        gc.collect()
        torch.cuda.empty_cache()
        toks = src.take(96)
        rows = {}
        for dt in ("float32", "bfloat16"):
            m2 = wl.random_model("8b", dt, dev, seed=0, layers=2)
            e2 = Engine(m2, EngineConfig(dtype=dt, max_model_len=256, kv_cache_tokens=256, enable_prefix_caching=False,
                                         warmup=False, cuda_graphs=False, sched=SchedulerConfig(max_num_seqs=1)))
            rc = e2.runner.manager.new_request()
            e2.runner.manager.allot_state(rc)
            assert e2.runner.manager.allocate(rc, 0, len(toks))
            rows[dt] = e2.runner.step([StepEntry(rc, toks, 0, [len(toks) - 1])]).float().cpu()
            del e2, m2
            gc.collect()
            torch.cuda.empty_cache()
        check = {"layers": 2, "tokens": len(toks), "max_abs_err_bf16_vs_fp32": (rows["float32"] - rows["bfloat16"]).abs().max().item(),
                 "logit_max_abs": rows["float32"].abs().max().item()}

        # ---- the continuous-batching workload at the Qwen3-0.6B shape (scheduler, prefix reuse, preemption, graphs) ----
        if not args.skip_serve:
            res = wl.serving_workload("0.6b", 256, device=dev)
            for k_ in ("total_tok_s", "gen_tok_s", "ttft_ms", "tpot_ms", "prefix_hit_rate", "preemptions", "kv_usage_peak",
                       "wall_s", "errors", "alone_identical", "alone_agreeing_token_share"):
                points[f"serve06b_{k_}"] = res[k_]
            gc.collect()
            torch.cuda.empty_cache()

        # ---- the Qwen3-32B shape: decode 1 / 8 / 64 from 2,048-token prompts, prefill of 2,048 tokens ---------
        if not args.skip_32b:
            m32 = wl.random_model("32b", "bfloat16", dev, seed=0)
            res = wl.decode_and_prefill_points(m32, (1, 8, 64), 2048, min(K, 32), W, (2048,), 4096, peaks,
                                               cuda_graphs=not args.no_cuda_graphs)
            for b, r in res["decode"].items():
                points[f"q32b_decode_b{b}"] = r["tokens_per_s"]
                points[f"q32b_decode_b{b}_hbm_frac"] = r["roofline_frac"]
            for t, r in res["prefill"].items():
                points[f"q32b_prefill_{t}"] = r["tokens_per_s"]
                points[f"q32b_prefill_{t}_frac"] = r["frac"]
            kern.tcgen05_check(dev)
            del res, m32
            gc.collect()
            torch.cuda.empty_cache()

    line = {
        "metric": "decode tokens/s (Qwen3-8B shape, batch 8)" if B == 8 else f"decode tokens/s (Qwen3-8B shape, batch {B})",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0, 0.02), uniform random token ids (seed 1234)",
        "config": {"model": "Qwen3-8B shape (BASELINE.json configs[2])", "global_batch": B, "seq_len": PROMPT_LEN,
                   "parallelism": "single GPU", "layers": cfg.num_hidden_layers, "layers_of_config": SHAPE_8B["num_hidden_layers"],
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "context_len": CONTEXT_LEN, "prompt_len": PROMPT_LEN, "decode_ctx_avg": ctx_avg, "kv_block": 16,
                   "cuda_graphs": not args.no_cuda_graphs, "l2": "inputs larger than L2 (15 GB of weights per step)",
                   "peaks": peak_kind},
        "e2e": e2e, "gpu_launches": int(launches), "clocks": sampler.summary(),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "bytes_per_step": bytes_step},
        "points": points,
    }
    if prefill is not None:
        line["prefill"] = prefill
    if check is not None:
        line["check"] = check
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
