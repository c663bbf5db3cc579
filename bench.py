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

# BASELINE.json configs[2]: Qwen3-8B shape
SHAPE_8B = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
                max_position_embeddings=40960, tie_word_embeddings=False)
CONTEXT_LEN = 8192          # the engine's max_model_len for the benchmark
PROMPT_LEN = 1024           # decode starts from prompts of this many random tokens
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                    "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"]))}, "measured"
        except (KeyError, ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0), "fallback"


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
    ap.add_argument("--skip-points", action="store_true", help="leave out the batch 1 / 64 points and the prefill")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "CocoRoF/iian is a C++/CMake program with no setup.py or "
                          "pyproject.toml (pip: 'not installable'), reads GGUF checkpoints only and has no sm_100 build; "
                          "there is nothing to install under baseline/_ref"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    K, W = args.steps, max(3, args.warmup)

    import torch
    from iian_b200 import EngineConfig, SamplingParams, SchedulerConfig
    from iian_b200 import ops
    from iian_b200.config.registry import get_architecture
    from iian_b200.engine.engine import Engine
    from iian_b200.engine.model import Model
    from iian_b200.engine.runner import StepEntry
    from iian_b200.models.qwen3 import qwen3_config_from_dict

    peaks, peak_kind = load_peaks()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    shape = dict(SHAPE_8B, num_hidden_layers=args.layers)
    cfg = qwen3_config_from_dict(shape)
    arch = get_architecture("Qwen3ForCausalLM")
    t_build = time.time()
    model = Model.from_random(arch, cfg, seed=0, dtype="bfloat16", device=dev, norm_jitter=0.0)
    max_b = max(args.batch, 1 if args.skip_points else 64)
    per_req = PROMPT_LEN + W + K + 48
    ecfg = EngineConfig(dtype="bfloat16", max_model_len=CONTEXT_LEN, kv_cache_tokens=max(CONTEXT_LEN, max_b * per_req),
                        block_size=16, enable_prefix_caching=False, warmup=True, cuda_graphs=not args.no_cuda_graphs,
                        sched=SchedulerConfig(max_num_seqs=max_b, max_num_batched_tokens=2048))
    engine = Engine(model, ecfg)
    runner, mgr, kern = engine.runner, engine.runner.manager, ops.kernels()
    print(f"[bench] model and engine ready in {time.time() - t_build:.1f} s "
          f"({model.weight_bytes / 1e9:.2f} GB of weights, cache {runner.storage.bytes / 1e9:.2f} GB)", file=sys.stderr)

    gen = torch.Generator().manual_seed(1234)
    def rand_tokens(n):
        return torch.randint(5, cfg.vocab_size - 5, (n,), generator=gen).tolist()

    layer_w = cfg.hidden_size * (cfg.q_size + 2 * cfg.kv_size) + cfg.q_size * cfg.hidden_size \
        + 3 * cfg.hidden_size * cfg.intermediate_size
    head_w = cfg.vocab_size * cfg.hidden_size
    weight_bytes_step = 2 * (cfg.num_hidden_layers * layer_w + head_w)
    kv_bytes_token = cfg.num_hidden_layers * 2 * cfg.kv_size * 2

    def prefill_requests(B):
        caches = []
        for _ in range(B):
            rc = mgr.new_request()
            mgr.allot_state(rc)
            caches.append(rc)
        prompts = [rand_tokens(PROMPT_LEN) for _ in range(B)]
        per_step = max(1, 2048 // PROMPT_LEN)
        for i in range(0, B, per_step):
            ents = []
            for rc, pr in zip(caches[i:i + per_step], prompts[i:i + per_step]):
                assert mgr.allocate(rc, 0, PROMPT_LEN)
                ents.append(StepEntry(rc, pr, 0, []))
            runner.step(ents)
        return caches

    def decode_device_timed(B, warm, steps):
        caches = prefill_requests(B)
        out = torch.empty(B, dtype=torch.int32, device=dev)
        toks = rand_tokens(B)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        pos = PROMPT_LEN
        launches0 = 0
        for i in range(warm + steps):
            if i == warm:
                torch.cuda.synchronize()
                launches0 = runner.launches
                start.record()
            ents = []
            for rc, t in zip(caches, toks):
                assert mgr.allocate(rc, pos, 1)
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
        ctx_avg = PROMPT_LEN + warm + (steps + 1) / 2
        return ms, launches, ctx_avg

    # ---- timed: decode at the headline batch (device clock) -------------------------------------
    sampler = ClockSampler(0)
    sampler.start()
    B = args.batch
    ms_step, launches, ctx_avg = decode_device_timed(B, W, K)
    value = B / (ms_step * 1e-3)
    bytes_step = weight_bytes_step + B * ctx_avg * kv_bytes_token
    achieved = bytes_step / (ms_step * 1e-3) / 1e9

    # ---- timed: the same through the Python entry point (host tokens in and out) -----------------
    sp = SamplingParams(temperature=0.0, max_tokens=W + K + 8, ignore_eos=True)
    reqs = [engine.submit(rand_tokens(PROMPT_LEN), sp) for _ in range(B)]
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

    points, prefill = {}, None
    if not args.skip_points:
        for b in (1, 64):
            ms_b, _, _ = decode_device_timed(b, W, K)
            points[f"decode_b{b}"] = b / (ms_b * 1e-3)
        # ---- prefill of one 2,048-token prompt --------------------------------------------------
        toks = rand_tokens(PREFILL_TOKENS)
        times = []
        for i in range(W + 5):
            rc = mgr.new_request()
            mgr.allot_state(rc)
            assert mgr.allocate(rc, 0, PREFILL_TOKENS)
            s_ev, e_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s_ev.record()
            runner.step([StepEntry(rc, toks, 0, [PREFILL_TOKENS - 1])])
            e_ev.record()
            torch.cuda.synchronize()
            if i >= W:
                times.append(s_ev.elapsed_time(e_ev))
            mgr.free(rc)
        p_ms = statistics.median(times)
        T = PREFILL_TOKENS
        flops = 2.0 * T * cfg.num_hidden_layers * layer_w + 2.0 * head_w \
            + cfg.num_hidden_layers * 4.0 * cfg.q_size * T * (T + 1) / 2
        prefill = {"value": T / (p_ms * 1e-3), "tokens": T, "ms": p_ms,
                   "frac": flops / (p_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), "tflops": flops / (p_ms * 1e-3) / 1e12}
    sampler.stop()
    if hasattr(kern, "tcgen05_check"):
        kern.tcgen05_check(dev)          # a tcgen05 kernel that gave up on a barrier would have left garbage

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
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
