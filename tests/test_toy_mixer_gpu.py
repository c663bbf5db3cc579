"""A toy architecture defined entirely in the tests (``tests/toy_model.py``), registered, built from a model
folder and stepped through the engine's own step function -- without a change to any file of the framework.

It has what Qwen3 does not: a mixer with a fixed-size state of its own per request, different mixers in
different layers, a layer that runs twice with a cache for each run, and a layer that reads the cache another
layer filled; a second layout has no attention and so needs no pages at all.  Here it is replayed under every
way of cutting the work, with and without CUDA graphs, and driven through the engine (scheduler, preemption,
shared prefixes, graphs) against the plain model.
"""
import json
import os

import pytest
import torch

from helpers import first_bad, random_tokens, replay_and_collect, trace_mixed, trace_portions, trace_tail, trace_whole
from iian_b200.parts.base import StateNeed
from toy_model import CFG, CFG_EMA_ONLY, CFG_PARALLEL, CFG_ROUTED, plain_toy, plain_toy_greedy, register_toy, unregister_toy, write_toy

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def toys(tmp_path_factory):
    register_toy()
    out = {"mixed": (write_toy(str(tmp_path_factory.mktemp("toy")), CFG), CFG),
           "ema_only": (write_toy(str(tmp_path_factory.mktemp("toy_ema")), CFG_EMA_ONLY, seed=10), CFG_EMA_ONLY),
           "routed": (write_toy(str(tmp_path_factory.mktemp("toy_routed")), CFG_ROUTED, seed=11), CFG_ROUTED),
           "parallel": (write_toy(str(tmp_path_factory.mktemp("toy_parallel")), CFG_PARALLEL, seed=12), CFG_PARALLEL)}
    yield out
    unregister_toy()


@pytest.fixture(scope="module")
def toy(toys):
    return toys["mixed"][0]


def test_toy_is_built_from_registered_parts(toy):
    from iian_b200.engine.model import Model
    m = Model.from_folder(toy, "float32", "cuda:0")
    assert m.graph_safe()
    assert m.arch.name == "ToyForCausalLM"
    assert [type(b.mixer).__name__ for b in m.blocks] == ["Attention", "ToyEma", "Attention"]
    needs = m.cache_needs()
    assert sorted(needs) == [0, 1, 2] and isinstance(needs[1], StateNeed) and needs[0] == needs[2]
    with open(os.path.join(toy, "config.json")) as f:
        assert json.load(f)["architectures"] == ["ToyForCausalLM"]


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("layout", ["mixed", "ema_only", "routed", "parallel"])
def test_toy_steps_like_its_plain_model(toys, layout, dtype, mode, graphs):
    """With ``graphs`` the decode-only steps are replayed from captured CUDA graphs: the state must advance
    exactly once per step (also on the step that captures a new graph)."""
    from iian_b200.engine.replay import TraceReplayer
    toy, cfg = toys[layout]
    if graphs and mode in ("whole", "portions"):
        pytest.skip("no step of this trace is decode-only")
    reqs = {f"r{i}": random_tokens(cfg["vocab_size"], n, 70 + i) for i, n in enumerate([3, 40, 21, 64, 9, 33])}
    want = {rid: plain_toy(toy, toks, cfg) for rid, toks in reqs.items()}
    steps = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions}.get(mode)
    steps = steps(reqs) if steps else trace_mixed(reqs, 192, seed=4, max_live=3)
    rp = TraceReplayer.from_folder(toy, dtype, 192, block_size=8, max_requests=3)     # 3 slots: they are used again
    assert rp.runner.native is None, "a model with parts of the test's own runs through the Python step function"
    rp.runner.cuda_graphs = graphs
    got = replay_and_collect(rp, steps)
    if graphs:
        assert rp.runner.num_graphs, "no decode graph was captured"
    scale = max(v.abs().max().item() for v in want.values())
    tol = 3e-5 * max(scale, 1.0) if dtype == "float32" else 2.5e-2 * scale
    if layout == "routed" and dtype == "bfloat16":
        # a token whose second and third best experts tie within rounding may be routed differently: allow a few rows
        bad_rows = [k for k in got if (got[k].double() - want[k[0]][k[1]]).abs().max().item() > tol]
        assert len(bad_rows) <= len(got) // 50, f"{len(bad_rows)} of {len(got)} rows beyond tolerance"
    else:
        bad = first_bad(got, want, tol)
        assert bad is None, f"first wrong logits at request {bad[0]} position {bad[1]} (err {bad[2]:.3g}, tol {tol:.3g})"
    assert len(got) == sum(len(t) for t in reqs.values())
    assert rp.runner.manager.slots.num_free == 3 and all(p.num_free == p.num_blocks for p in rp.runner.manager.pools)


def test_a_model_without_pages_builds_and_runs(toys):
    """No mixer of the EMA-only layout keeps keys: the cache manager has no page group, requests hold a state
    slot only, and prefix reuse is off because a state cannot be shared page by page."""
    from iian_b200.engine.model import Model
    from iian_b200.engine.runner import ModelRunner
    d, cfg = toys["ema_only"]
    m = Model.from_folder(d, "float32", "cuda:0")
    assert all(isinstance(n, StateNeed) for n in m.cache_needs().values())
    r = ModelRunner(m, block_size=8, capacity_tokens=64, max_num_seqs=2, enable_prefix_caching=True)
    assert r.manager.groups == [] and not r.prefix_caching and r.manager.usage == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layout", ["mixed", "ema_only"])
def test_toy_through_the_engine_with_graphs_prefixes_and_preemption(toys, layout, dtype):
    """The engine's defaults (CUDA graphs on, prefix reuse asked for) with a model that keeps state: prompts that
    share a prefix, so few pages that requests are preempted and resumed, greedy tokens against the plain model.
    Prefix reuse must have been switched off (a hit would skip tokens the state needs); graphs must be in use."""
    from iian_b200 import EngineConfig, SchedulerConfig
    from iian_b200.engine.engine import Engine
    d, cfg = toys[layout]
    v = cfg["vocab_size"]
    shared = random_tokens(v, 24, 5)
    prompts = [shared + random_tokens(v, n, 20 + i) for i, n in enumerate([3, 9, 17, 30])] + [random_tokens(v, 5, 99)]
    n_new = 20
    want = [plain_toy_greedy(d, p, n_new, cfg) for p in prompts]
    for kv_tokens in (1024, 96):                     # ample pages; then so few that the scheduler preempts
        eng = Engine(d, EngineConfig(dtype=dtype, block_size=8, max_model_len=96, kv_cache_tokens=kv_tokens,
                                     enable_prefix_caching=True, cuda_graphs=True,
                                     sched=SchedulerConfig(max_num_batched_tokens=32, max_num_seqs=4)))
        assert eng.runner.cuda_graphs and not eng.runner.prefix_caching
        for rounds in range(2):                      # the second round would hit the prefixes of the first
            got = eng.generate(prompts, max_tokens=n_new, temperature=0.0)
            for g, (wt, margins) in zip(got, want):
                for k, (a, b) in enumerate(zip(g, wt)):
                    if a != b:
                        assert dtype == "bfloat16" and margins[k] < 0.05, f"{layout} token {k}: {g} vs {wt} (margin {margins[k]:.4f})"
                        break
                else:
                    assert len(g) == len(wt)
        assert eng.runner.num_graphs, "no decode graph was captured"
        assert eng.stats().prefix_cache_hits == 0
        if kv_tokens == 96 and layout == "mixed":
            assert eng.stats().preemptions >= 1
        eng.cache.check_invariants()
        assert eng.cache.slots.num_free == eng.cache.slots.num_slots
