"""Generation through the Python entry point and the command line on the GPU: greedy tokens equal the
plain implementation's (alone, batched, with chunked prefill, with preemption, with prefix reuse, with
and without CUDA graphs); sampled tokens follow the plain sampling walk with the request's own stream of
uniform numbers and do not depend on what else runs."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen3 as plain
from helpers import BLOCK_SIZE, TINY, random_tokens, write_tiny

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_MASK = (1 << 64) - 1


def splitmix64(x):
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def stream(seed, i):
    """Number i of a request's stream of uniforms, written out here independently of the engine."""
    h = splitmix64(splitmix64(seed & _MASK) ^ ((i * 0xD1B54A32D192ED03) & _MASK))
    return (h >> 40) / float(1 << 24)


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    root = tmp_path_factory.mktemp("m")
    out = {}
    for name in sorted(TINY):
        d = write_tiny(root, name, store_dtype=torch.bfloat16)
        cfg, w = plain.load_folder(d)
        out[name] = (d, cfg, w)
    return out


def plain_greedy(cfg, w, prompt, n):
    toks, margins = list(prompt), []
    for _ in range(n):
        row = plain.forward(cfg, w, toks)[-1]
        top = torch.topk(row, 2).values
        margins.append((top[0] - top[1]).item())
        toks.append(plain.argmax(row))
    return toks[len(prompt):], margins


def assert_tokens(got, want, margins, dtype, what):
    """Token by token up to the first near-tie: in bfloat16 a request is checked only as far as its first token
    whose two best logits lie within the margin; what follows a legitimately different token is not compared."""
    for k, (a, b) in enumerate(zip(got, want)):
        if a != b:
            # bfloat16 may take the runner-up of a near tie (the reference accepts the same on GPUs,
            # tests/e2e/test-batching.cpp:34-77); after that the sequences legitimately differ
            assert dtype == "bfloat16" and margins[k] < 0.02, f"{what}: token {k}: {got} vs {want} (margin {margins[k]:.4f})"
            return
    assert len(got) == len(want)


def make_engine(d, dtype, name, **kw):
    from iian_b200 import EngineConfig, SchedulerConfig
    from iian_b200.engine.engine import Engine
    sched = SchedulerConfig(max_num_batched_tokens=kw.pop("budget", 1024), max_num_seqs=kw.pop("seqs", 8))
    return Engine(d, EngineConfig(dtype=dtype, block_size=BLOCK_SIZE[name], sched=sched, **kw))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
def test_greedy_generation_through_the_entry_point(setup, name, dtype):
    d, cfg, w = setup[name]
    v = TINY[name]["vocab_size"]
    lengths = [5, 17, 33] if name == "A" else [1, 7, 24, 61, 100]
    n_new = 8 if name == "A" else 12
    prompts = [random_tokens(v, n, 1 + i) for i, n in enumerate(lengths)]
    want = [plain_greedy(cfg, w, p, n_new) for p in prompts]
    max_len = min(TINY[name]["max_position_embeddings"], 256)
    variants = [dict(budget=1024, kv_cache_tokens=4 * max_len, enable_prefix_caching=False),
                dict(budget=13, kv_cache_tokens=4 * max_len, enable_prefix_caching=True),        # chunked prefill, mixed steps
                dict(budget=64, kv_cache_tokens=max_len, enable_prefix_caching=False),            # few pages: preemption
                dict(budget=1024, kv_cache_tokens=4 * max_len, cuda_graphs=False)]
    for kw in variants:
        eng = make_engine(d, dtype, name, max_model_len=max_len, **kw)
        got = eng.generate(prompts, max_tokens=n_new, temperature=0.0)
        for g, (wt, margins) in zip(got, want):
            assert_tokens(g, wt, margins, dtype, f"{name} {kw}")
        again = eng.generate(prompts, max_tokens=n_new, temperature=0.0)      # the second time some prefixes are cached
        if dtype == "float32":
            assert again == got
        else:       # a prefix hit cuts the prompt differently, and in bfloat16 another cut rounds differently
            for g, (wt, margins) in zip(again, want):
                assert_tokens(g, wt, margins, dtype, f"{name} {kw} (second time)")
        eng.cache.check_invariants()
        assert all(p.num_free == p.num_blocks for p in eng.cache.pools)
        if kw.get("kv_cache_tokens") == max_len and name != "A":
            assert eng.stats().preemptions >= 1


def test_temperature_sampling_follows_the_plain_walk(setup):
    """Configuration B of the baseline workload: prompts 1/7/24/61/100, portions of 13, 12 new tokens at
    temperature 0.7, sampler seed 4.  In float32 every sampled token must be the one the plain walk
    picks for the request's i-th uniform number (unless that number falls within rounding of an edge)."""
    from iian_b200 import SamplingParams
    d, cfg, w = setup["B"]
    prompts = [random_tokens(503, n, 3 + i) for i, n in enumerate([1, 7, 24, 61, 100])]
    eng = make_engine(d, "float32", "B", budget=13, kv_cache_tokens=1024, max_model_len=256)
    reqs = [eng.submit(p, SamplingParams(temperature=0.7, seed=4 + i, max_tokens=12)) for i, p in enumerate(prompts)]
    while any(not r.is_finished for r in reqs):
        eng.step()
    for i, r in enumerate(reqs):
        toks = list(prompts[i])
        for k, tok in enumerate(r.output_tokens):
            probs = plain.candidate_probs(plain.forward(cfg, w, toks)[-1].float(), 0.7)
            u = stream(4 + i, k)
            want = plain.sample_from(probs, u)
            if tok != want:
                cum = torch.cumsum(probs, 0)
                target = u * cum[-1].item()
                edge = min(abs(cum[tok].item() - target), abs(cum[tok].item() - probs[tok].item() - target))
                assert edge < 1e-5 * cum[-1].item(), f"request {i} token {k}: engine {tok}, plain {want}"
            toks.append(tok)
    # the same request alone, with another budget and top-k/top-p/min-p off and on: same seed, same tokens
    alone = make_engine(d, "float32", "B", budget=64, kv_cache_tokens=1024, max_model_len=256)
    r = alone.submit(prompts[3], SamplingParams(temperature=0.7, seed=7, max_tokens=12))
    while not r.is_finished:
        alone.step()
    assert r.output_tokens == reqs[3].output_tokens, "a request's tokens must not depend on what else runs"
    r2 = alone.submit(prompts[3], SamplingParams(temperature=0.7, seed=7, max_tokens=12, top_k=1))
    while not r2.is_finished:
        alone.step()
    greedy, _ = plain_greedy(cfg, w, prompts[3], 12)
    assert r2.output_tokens == greedy, "top_k = 1 is greedy"


@pytest.mark.parametrize("name", ["B", "D"])
def test_temperature_sampling_with_graphs_few_pages_and_shared_prefixes(setup, name):
    """Sampling, CUDA-graph decode, preemption and prefix reuse together: in float32 every sampled token is still the
    one the plain walk picks for the request's i-th uniform number, although requests are cut into portions, thrown
    out for lack of pages and recomputed, start behind a cached prefix, and decode from replayed graphs."""
    from iian_b200 import SamplingParams
    d, cfg, w = setup[name]
    v, bs = cfg["vocab_size"], BLOCK_SIZE[name]
    shared = random_tokens(v, 2 * bs + 3, 500)
    prompts = [shared + random_tokens(v, 4 + 7 * i, 510 + i) if i % 2 else random_tokens(v, 9 + 11 * i, 520 + i) for i in range(6)]
    longest = max(len(p) for p in prompts) + 12
    kv = -(-longest // bs) * bs + 2 * bs                                  # room for one long request and little more
    eng = make_engine(d, "float32", name, budget=17, seqs=6, kv_cache_tokens=kv, max_model_len=kv, enable_prefix_caching=True,
                      cuda_graphs=True)
    reqs = [eng.submit(p, SamplingParams(temperature=0.8, seed=30 + i, max_tokens=12, ignore_eos=True)) for i, p in enumerate(prompts)]
    for _ in range(5000):
        if all(r.is_finished for r in reqs):
            break
        eng.step()
    assert all(r.is_finished and len(r.output_tokens) == 12 for r in reqs)
    st = eng.stats()
    assert st.preemptions >= 1 and st.prefix_cache_hits >= 1 and eng.runner.num_graphs >= 1
    for i, r in enumerate(reqs):
        toks = list(prompts[i])
        for k, tok in enumerate(r.output_tokens):
            probs = plain.candidate_probs(plain.forward(cfg, w, toks)[-1].float(), 0.8)
            u = stream(30 + i, k)
            want = plain.sample_from(probs, u)
            if tok != want:
                cum = torch.cumsum(probs, 0)
                target = u * cum[-1].item()
                edge = min(abs(cum[tok].item() - target), abs(cum[tok].item() - probs[tok].item() - target))
                assert edge < 1e-5 * cum[-1].item(), f"request {i} token {k}: engine {tok}, plain {want}"
            toks.append(tok)
    assert all(p.num_free == p.num_blocks for p in eng.cache.pools)


def _collect_logits(eng):
    """(request id, position) -> the logits row the engine sampled that position's next token from."""
    rows = {}

    def hook(reqs, logits):
        host = logits.detach().float().cpu()
        for i, r in enumerate(reqs):
            rows[(r.id, r.n_tokens - 1)] = host[i].clone()
    eng.logits_hook = hook
    return rows


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D", "E"])
def test_logits_under_the_scheduler_with_graphs_prefix_hits_and_preemption(setup, name, dtype):
    """Twelve requests live at once (graphs for padded batches of 16), half of them behind a shared prefix
    (prefix reuse on), so few pages that requests are preempted and resumed: every row of logits a token was
    sampled from is compared with the plain implementation on that request's own tokens -- logits, not tokens,
    so a near-tie does not end the comparison."""
    from iian_b200 import SamplingParams
    d, cfg, w = setup[name]
    v = TINY[name]["vocab_size"]
    bs = BLOCK_SIZE[name]
    shared = random_tokens(v, 3 * bs + 5, 200)
    prompts = []
    for i in range(12):
        tail = random_tokens(v, 2 + (7 * i) % 23, 210 + i)
        prompts.append(shared + tail if i % 2 == 0 else tail + random_tokens(v, 10 + i, 230 + i))
    eng = make_engine(d, dtype, name, seqs=16, budget=48, max_model_len=128, kv_cache_tokens=384,
                      enable_prefix_caching=True, cuda_graphs=True)
    rows = _collect_logits(eng)
    temp = 0.8 if dtype == "float32" else 0.0
    reqs = [eng.submit(p, SamplingParams(temperature=temp, seed=50 + i, max_tokens=14, ignore_eos=True)) for i, p in enumerate(prompts)]
    while any(not r.is_finished for r in reqs):
        eng.step()
    st = eng.stats()
    assert st.preemptions >= 1 and st.prefix_cache_hits >= 1 and eng.runner.num_graphs
    worst = 0.0
    for i, r in enumerate(reqs):
        assert r.n_output == 14
        full = plain.forward(cfg, w, r.tokens)
        scale = full.abs().max().item()
        tol_ = 2e-5 * max(1.0, scale) if dtype == "float32" else 2.5e-2 * scale
        for k in range(14):
            pos = r.n_prompt + k - 1
            err = (rows[(r.id, pos)].double() - full[pos]).abs().max().item()
            worst = max(worst, err / tol_)
            assert err <= tol_, f"request {i} position {pos}: logits differ by {err:.3g} (tol {tol_:.3g})"
            if temp > 0:          # and the sampled token is the plain walk's for the request's k-th uniform number
                probs = plain.candidate_probs(full[pos].float(), temp)
                u = stream(50 + i, k)
                want = plain.sample_from(probs, u)
                tok = r.tokens[r.n_prompt + k]
                if tok != want:
                    cum = torch.cumsum(probs, 0)
                    target = u * cum[-1].item()
                    edge = min(abs(cum[tok].item() - target), abs(cum[tok].item() - probs[tok].item() - target))
                    assert edge < 1e-4 * cum[-1].item(), f"request {i} token {k}: engine {tok}, plain {want}"
    print(f"[{name} {dtype}] worst error / tolerance {worst:.3f}; preemptions {st.preemptions}, prefix hits {st.prefix_cache_hits}")
    eng.cache.check_invariants()
    assert all(p.num_free == p.num_blocks for p in eng.cache.pools)


def test_command_line(setup, tmp_path):
    d, cfg, w = setup["B"]
    prompt = random_tokens(503, 9, 77)
    want, _ = plain_greedy(cfg, w, prompt, 5)
    exe = os.path.join(ROOT, "bin", "iian")
    proc = subprocess.run([sys.executable, exe, "complete", d, "-p", ",".join(map(str, prompt)), "-n", "5", "--temp", "0",
                           "--dtype", "float32", "--block-size", "8", "--json", "-q"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-1500:]
    out = json.loads(proc.stdout)
    assert out["tokens"] == want and out["completion_tokens"] == 5 and out["finish_reason"] == "length"
    proc = subprocess.run([sys.executable, exe, "bench", d, "--concurrency", "1,3", "--prompt-tokens", "20", "--gen-tokens", "4",
                           "--json", "--block-size", "8"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-1500:]
    rows = json.loads(proc.stdout)
    assert [r["concurrency"] for r in rows] == [1, 3] and all(r["gen_tps"] > 0 and r["ttft_ms"] > 0 for r in rows)
    proc = subprocess.run([sys.executable, exe, "complete", str(tmp_path), "-p", "1"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 1 and "config.json" in proc.stderr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C", "D", "E", "F"])
def test_decode_steps_from_graphs_match_eager_steps(setup, name, dtype):
    """Decode-only steps replayed from captured graphs (padded batch, buffers kept between steps, block-table
    rows only appended to) against the same steps run eagerly: requests leave, a new one takes a freed row,
    the order of the batch changes, pages fill up and new ones are taken, a freed request's cache object
    comes back with other pages."""
    from iian_b200.engine.model import Model
    from iian_b200.engine.replay import TraceReplayer
    d, cfg, w = setup[name]
    v = TINY[name]["vocab_size"]
    bs = BLOCK_SIZE[name]
    model = Model.from_folder(d, dtype, "cuda:0")
    reps = [TraceReplayer(model, 1024, bs, 8), TraceReplayer(model, 1024, bs, 8)]
    reps[1].runner.cuda_graphs = True
    prompts = {k: random_tokens(v, n, 40 + i) for i, (k, n) in enumerate([("a", 2 * bs - 1), ("b", 5), ("c", 3 * bs), ("d", bs + 2)])}
    script, step = [], 0
    for k in ("a", "b", "c"):                                   # whole prompts, one step each
        script.append({"step": step, "entries": [{"id": k, "tokens": prompts[k], "want": [len(prompts[k]) - 1]}], "end": []})
        step += 1
    nxt = {k: random_tokens(v, 6 * bs + 40, 90 + i) for i, k in enumerate("abcd")}
    used = {k: 0 for k in "abcd"}

    def decode(ids, end=()):
        nonlocal step
        ents = []
        for k in ids:
            ents.append({"id": k, "tokens": [nxt[k][used[k]]], "want": [0]})
            used[k] += 1
        script.append({"step": step, "entries": ents, "end": list(end)})
        step += 1

    for _ in range(bs + 2):
        decode("abc")
    decode("abc", end="b")
    for _ in range(3):
        decode("ac")
    script.append({"step": step, "entries": [{"id": "d", "tokens": prompts["d"], "want": [len(prompts["d"]) - 1]}], "end": []})
    step += 1
    for _ in range(bs):
        decode("dac")
    decode("cda", end="a")
    script.append({"step": step, "entries": [{"id": "a", "tokens": prompts["b"], "want": [4]}], "end": []})   # "a" again, new pages
    step += 1
    for _ in range(4):
        decode("acd")
    tol_ = 1e-5 if dtype == "float32" else 0.05
    for rec in script:
        outs = [r.run_step(rec) for r in reps]
        if outs[0] is None:
            assert outs[1] is None
            continue
        err = (outs[0].float() - outs[1].float()).abs().max().item()
        scale = max(1.0, outs[0].float().abs().max().item())
        assert err <= tol_ * scale, f"step {rec['step']}: graph and eager logits differ by {err} (scale {scale})"
    assert reps[1].runner.num_graphs, "no decode graph was captured"


def test_product_dispatch_by_tiles(monkeypatch):
    """bfloat16 products: up to 8 rows the weight-streaming kernel, from 128 rows the tcgen05 kernel if the product
    has several waves of tiles of 256 x 256, the library product in between and for fewer tiles."""
    from iian_b200.ops.cuda_backend import CudaKernels
    k = CudaKernels()
    monkeypatch.setattr(CudaKernels, "TCGEN05_MIN_TILES", 300)
    def ok(rows, out_features, in_features=4096):
        x = torch.empty(rows, in_features, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(out_features, in_features, dtype=torch.bfloat16, device="cuda")
        return k._tcgen05_ok(x, w, rows, in_features), k.can_fuse_norm(x, w), k.can_take_prenormed(rows, w, torch.bfloat16)
    assert ok(8, 4096) == (False, True, True)               # the streaming kernel folds norms too
    assert ok(64, 4096) == (False, False, False)
    assert ok(2048, 4096) == (False, False, False)          # 8 x 16 tiles: the library
    assert ok(2048, 6144) == (False, False, False)          # 8 x 24
    assert ok(1024, 24576) == (True, True, True)            # 4 x 96
    assert ok(512, 24576) == (False, False, False)          # 2 x 96
    assert ok(2048, 151936)[0]
