"""The engine above the step function, on the CPU with the torch stand-in for the kernels: greedy
generation equals the plain implementation's, with chunked prefill, with so few pages that requests
are preempted and resumed, and with prefix reuse; finish rules; errors at submission."""
import pytest
import torch

import plain_qwen3 as plain
from fake_kernels import FakeKernels
from helpers import TINY, random_tokens, write_tiny
from iian_b200 import EngineConfig, SamplingParams, SchedulerConfig, ops
from iian_b200.engine.engine import Engine
from iian_b200.engine.model import Model
from iian_b200.engine.request import FinishReason


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    d = write_tiny(tmp_path_factory.mktemp("m"), "B")
    cfg, w = plain.load_folder(d)
    prompts = [random_tokens(503, n, 100 + i) for i, n in enumerate([1, 7, 24, 61])]

    def greedy(prompt, n):
        toks = list(prompt)
        for _ in range(n):
            toks.append(plain.argmax(plain.forward(cfg, w, toks)[-1]))
        return toks[len(prompt):]
    want = [greedy(p, 6) for p in prompts]
    with ops.use_kernels(FakeKernels()):
        model = Model.from_folder(d, "float32", "cpu")
    return model, prompts, want


def engine(model, **kw):
    sched = SchedulerConfig(max_num_batched_tokens=kw.pop("budget", 13), max_num_seqs=kw.pop("seqs", 4))
    return Engine(model, EngineConfig(dtype="float32", block_size=8, warmup=False, sched=sched, **kw))


def test_greedy_generation_with_chunked_prefill(setup):
    model, prompts, want = setup
    with ops.use_kernels(FakeKernels()):
        eng = engine(model, kv_cache_tokens=256, max_model_len=128)
        assert eng.generate(prompts, max_tokens=6, temperature=0.0) == want
        st = eng.stats()
    assert st.requests_finished == 4 and st.generation_tokens == 24 and st.prompt_tokens == 93 and st.preemptions == 0
    eng.cache.check_invariants()
    assert all(p.num_free == p.num_blocks for p in eng.cache.pools)


def test_preempted_requests_resume_with_the_same_tokens(setup):
    model, prompts, want = setup
    with ops.use_kernels(FakeKernels()):
        eng = engine(model, kv_cache_tokens=96, max_model_len=96, budget=16, enable_prefix_caching=False)
        assert eng.generate(prompts, max_tokens=6, temperature=0.0) == want
        assert eng.stats().preemptions >= 1
    eng.cache.check_invariants()


def test_prefix_reuse_changes_nothing_but_the_work(setup):
    model, prompts, want = setup
    with ops.use_kernels(FakeKernels()):
        eng = engine(model, kv_cache_tokens=512, max_model_len=128, enable_prefix_caching=True)
        assert eng.generate(prompts, max_tokens=6, temperature=0.0) == want
        assert eng.stats().prefix_cache_hits == 0
        assert eng.generate(prompts, max_tokens=6, temperature=0.0) == want
        st = eng.stats()
    assert st.prefix_cache_hits == (24 - 1) // 8 + (61 - 1) // 8          # the last token is always computed
    assert st.cached_prompt_tokens == 8 * st.prefix_cache_hits


def test_finish_rules(setup):
    model, prompts, want = setup
    with ops.use_kernels(FakeKernels()):
        eng = engine(model, kv_cache_tokens=256, max_model_len=32)
        r = eng.submit(prompts[1], SamplingParams(temperature=0.0, max_tokens=3))
        while not r.is_finished:
            eng.step()
        assert r.output_tokens == want[1][:3] and r.finish_reason == FinishReason.LENGTH
        assert r.outputs[-1].finished and sum(len(c.tokens) for c in r.outputs) == 3
        k = next(i for i in range(1, 6) if want[1][i] not in want[1][:i])      # a token that first shows up at place k
        stop_at = want[1][k]
        r = eng.submit(prompts[1], SamplingParams(temperature=0.0, max_tokens=6, stop_token_ids=[stop_at]))
        while not r.is_finished:
            eng.step()
        assert r.output_tokens == want[1][:k + 1] and r.finish_reason == FinishReason.STOP and r.stop_reason == str(stop_at)
        r = eng.submit(prompts[2], SamplingParams(temperature=0.0))      # no max_tokens: stops when the context is full
        while not r.is_finished:
            eng.step()
        assert r.n_tokens == 32 and r.finish_reason == FinishReason.LENGTH
        r = eng.submit(prompts[2], SamplingParams(temperature=0.0, max_tokens=50))
        eng.step()
        eng.abort(r.id)
        eng.step()
        assert r.is_finished and r.finish_reason == FinishReason.ABORT
    assert all(p.num_free == p.num_blocks for p in eng.cache.pools)


def test_submission_errors(setup):
    model, prompts, _ = setup
    with ops.use_kernels(FakeKernels()):
        eng = engine(model, kv_cache_tokens=256, max_model_len=32)
        with pytest.raises(ValueError, match="empty"):
            eng.submit([])
        with pytest.raises(ValueError, match="out of range"):
            eng.submit([1, 503])
        with pytest.raises(ValueError, match="too long"):
            eng.submit(list(range(32)))
        with pytest.raises(ValueError, match="temperature"):
            eng.submit([1], SamplingParams(temperature=-1.0))
        with pytest.raises(ValueError, match="top_p"):
            eng.submit([1], SamplingParams(top_p=0.0))
        with pytest.raises(ValueError, match="max_model_len"):
            engine(model, kv_cache_tokens=16, max_model_len=64)


def test_a_request_that_cannot_fit_is_failed_not_hung(setup):
    model, prompts, _ = setup
    with ops.use_kernels(FakeKernels()):
        eng = engine(model, kv_cache_tokens=64, max_model_len=64, budget=64)
        a = eng.submit(prompts[3][:60], SamplingParams(temperature=0.0, max_tokens=2))
        b = eng.submit(prompts[3][:60], SamplingParams(temperature=0.0, max_tokens=2))
        for _ in range(40):
            if a.is_finished and b.is_finished:
                break
            eng.step()
        assert a.is_finished and b.is_finished
        assert {a.finish_reason, b.finish_reason} <= {FinishReason.LENGTH, FinishReason.ERROR}
        assert FinishReason.LENGTH in {a.finish_reason, b.finish_reason}     # one after the other they both fit


def test_max_model_len_beyond_the_models_positions_is_refused(setup):
    model, _, _ = setup
    with ops.use_kernels(FakeKernels()):
        with pytest.raises(ValueError, match="positions"):
            engine(model, kv_cache_tokens=1024, max_model_len=TINY["B"]["max_position_embeddings"] + 1)


@pytest.mark.parametrize("layout", ["mixed", "ema_only"])
def test_a_model_with_state_runs_without_prefix_reuse(tmp_path, layout):
    """A mixer with a fixed-size state of its own (tests/toy_model.py): the engine is asked for prefix reuse
    and switches it off, because a request that started behind a cached prefix would lack the state those
    tokens build; with so few pages that requests are preempted, the tokens still equal the plain model's.
    The layout without attention has no page group at all."""
    from toy_model import CFG, CFG_EMA_ONLY, plain_toy_greedy, register_toy, unregister_toy, write_toy
    cfg = CFG if layout == "mixed" else CFG_EMA_ONLY
    register_toy()
    try:
        d = write_toy(str(tmp_path), cfg)
        v = cfg["vocab_size"]
        shared = random_tokens(v, 24, 5)
        prompts = [shared + random_tokens(v, n, 20 + i) for i, n in enumerate([3, 9, 17])]
        want = [plain_toy_greedy(d, p, 6, cfg)[0] for p in prompts]
        with ops.use_kernels(FakeKernels()):
            model = Model.from_folder(d, "float32", "cpu")
            eng = engine(model, kv_cache_tokens=64, max_model_len=64, budget=16, seqs=3, enable_prefix_caching=True)
            assert not eng.runner.prefix_caching
            assert len(eng.cache.groups) == (1 if layout == "mixed" else 0)
            for _ in range(2):
                assert eng.generate(prompts, max_tokens=6, temperature=0.0) == want
            st = eng.stats()
        assert st.prefix_cache_hits == 0
        if layout == "mixed":
            assert st.preemptions >= 1
        eng.cache.check_invariants()
        assert eng.cache.slots.num_free == eng.cache.slots.num_slots
    finally:
        unregister_toy()
