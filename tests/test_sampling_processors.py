"""The logits processors: the lists the sampler prepares (allowed ids and one edit per touched token) give, applied
to a dense row, what the plain implementation gives; on the GPU the kernel applies them, and generation with
penalties follows a plain walk."""
import random

import pytest
import torch

import plain_qwen3 as plain
from iian_b200.sampling.params import SamplingParams
from iian_b200.sampling.sampler import row_edits


def random_case(rng, vocab):
    prompt = [rng.randrange(vocab) for _ in range(rng.randrange(0, 12))]
    output = [rng.randrange(vocab) for _ in range(rng.randrange(0, 20))]
    kw = dict(presence=rng.choice([0.0, 0.7, -1.5]), frequency=rng.choice([0.0, 0.3, 2.0]),
              repetition=rng.choice([1.0, 1.3, 0.8]), last_n=rng.choice([-1, 0, 3, 50]))
    allowed = sorted(rng.sample(range(vocab), rng.randrange(1, vocab // 2))) if rng.random() < 0.3 else []
    bias = {rng.randrange(vocab): rng.uniform(-5, 5) for _ in range(rng.randrange(0, 4))}
    bad = []
    for _ in range(rng.randrange(0, 4)):
        n = rng.randrange(1, 4)
        if rng.random() < 0.6 and len(output) >= n - 1:      # one that matches the end of the output
            bad.append((output[len(output) - (n - 1):] if n > 1 else []) + [rng.randrange(vocab)])
        else:
            bad.append([rng.randrange(vocab) for _ in range(n)])
    banned = [rng.randrange(vocab)] if rng.random() < 0.3 else []
    p = SamplingParams(presence_penalty=kw["presence"], frequency_penalty=kw["frequency"],
                       repetition_penalty=kw["repetition"], repetition_last_n=kw["last_n"], logit_bias=bias,
                       allowed_token_ids=allowed, bad_words=bad)
    return p, prompt, output, banned, dict(allowed=allowed, bias=bias, bad_words=bad, banned=banned, **kw)


def apply_dense(logits, allowed, edits):
    l = logits.clone().double()
    if allowed:
        keep = torch.full_like(l, float("-inf"))
        keep[allowed] = l[allowed]
        l = keep
    for t, (pre, mp, mn, post) in edits.items():
        x = l[t] + pre
        x = x * mp if x > 0 else x * mn
        l[t] = x + post
    return l


@pytest.mark.parametrize("seed", range(40))
def test_row_edits_equal_the_plain_processors(seed):
    rng = random.Random(seed)
    vocab = 37
    p, prompt, output, banned, kw = random_case(rng, vocab)
    p.validate(vocab)
    logits = torch.randn(vocab, generator=torch.Generator().manual_seed(seed), dtype=torch.float64) * 3
    allowed, edits = row_edits(p, prompt, output, banned)
    got = apply_dense(logits, allowed, edits)
    want = plain.process_logits(logits, prompt, output, **kw)
    both_inf = torch.isinf(got) & torch.isinf(want)
    assert torch.equal(torch.isinf(got), torch.isinf(want))
    assert (got[~both_inf] - want[~both_inf]).abs().max() < 1e-12


def test_validation_of_penalties():
    with pytest.raises(ValueError, match="presence_penalty"):
        SamplingParams(presence_penalty=2.5).validate(10)
    with pytest.raises(ValueError, match="frequency_penalty"):
        SamplingParams(frequency_penalty=-3).validate(10)
    with pytest.raises(ValueError, match="repetition_penalty"):
        SamplingParams(repetition_penalty=0.0).validate(10)
    with pytest.raises(ValueError, match="logit_bias"):
        SamplingParams(logit_bias={10: 1.0}).validate(10)
    assert not SamplingParams().has_processors


@pytest.mark.gpu
def test_logit_edits_kernel():
    from iian_b200.sampling.sampler import Sampler
    rng = random.Random(7)
    vocab, rows = 1031, 6
    g = torch.Generator().manual_seed(3)
    logits = (torch.randn(rows, vocab, generator=g) * 3).float()
    cases = [random_case(rng, vocab) for _ in range(rows)]
    cases[2] = (SamplingParams(), [], [], [], dict())               # a row nothing happens to
    dev = logits.cuda()
    Sampler(dev.device).apply_processors(dev, [c[0] for c in cases], [(c[1], c[2]) for c in cases], [c[3] for c in cases])
    got = dev.cpu().double()
    for r, c in enumerate(cases):
        want = plain.process_logits(logits[r].double(), c[1], c[2], **c[4]) if c[4] else logits[r].double()
        assert torch.equal(torch.isinf(got[r]), torch.isinf(want)), r
        fin = ~torch.isinf(want)
        assert (got[r][fin] - want[fin]).abs().max() < 1e-5, r


@pytest.mark.gpu
def test_generation_with_penalties_follows_the_plain_walk(tmp_path):
    """Greedy generation in float32 with a repetition and a frequency penalty, a logit bias, a bad word and allowed
    ids: the engine's tokens are those of the plain model walked with the plain processors."""
    from helpers import TINY, random_tokens, write_tiny
    from iian_b200 import EngineConfig, SamplingParams as SP
    from iian_b200.engine.engine import Engine
    d = write_tiny(str(tmp_path), "A")
    cfg, w = plain.load_folder(d)
    vocab = TINY["A"]["vocab_size"]
    prompt = random_tokens(vocab, 9, 5)
    allowed = list(range(0, vocab, 2)) + [1, 3]
    kw = dict(allowed=allowed, bias={4: 1.5, 6: -2.0}, bad_words=[[8], [2, 10]], presence=0.4, frequency=0.9,
              repetition=1.4, last_n=5)
    toks, want, margins = list(prompt), [], []
    for _ in range(10):
        l = plain.process_logits(plain.forward(cfg, w, toks)[-1], prompt, toks[len(prompt):], **kw)
        top = torch.topk(l, 2).values
        margins.append(float(top[0] - top[1]))
        want.append(plain.argmax(l))
        toks.append(want[-1])
    eng = Engine(d, EngineConfig(dtype="float32", block_size=8, max_model_len=64, kv_cache_tokens=256))
    sp = SP(temperature=0.0, max_tokens=10, ignore_eos=True, presence_penalty=0.4, frequency_penalty=0.9,
            repetition_penalty=1.4, repetition_last_n=5, logit_bias={4: 1.5, 6: -2.0}, allowed_token_ids=allowed,
            bad_words=[[8], [2, 10]])
    r = eng.submit(prompt, sp)
    while not r.is_finished:
        eng.step()
    got = r.output_tokens
    for k, (a, b) in enumerate(zip(got, want)):
        if a != b:
            assert margins[k] < 1e-4, (k, got, want)
            break
    assert len(got) == 10 and 8 not in got and all(t in allowed for t in got)


@pytest.mark.gpu
def test_logprobs_kernel():
    from iian_b200.sampling.sampler import Sampler
    vocab, rows = 1500, 5
    g = torch.Generator().manual_seed(11)
    logits = (torch.randn(rows, vocab, generator=g) * 4).float()
    logits[1, 7] = logits[1, 900] = logits[1].max() + 1.0          # equal values: the lower id comes first
    logits[3, 10:20] = float("-inf")
    tokens = [3, 900, 55, 12, 1499]
    params = [SamplingParams(logprobs=k) for k in (0, 5, -1, 20, 1)]
    got = Sampler(torch.device("cuda")).logprobs(logits.cuda(), tokens, params)
    ref = torch.log_softmax(logits.double(), dim=-1)
    for r, p in enumerate(params):
        if p.logprobs < 0:
            assert got[r] is None
            continue
        lp, top = got[r]
        want_lp = ref[r, tokens[r]].item()
        assert lp == want_lp if want_lp == float("-inf") else abs(lp - want_lp) < 1e-4
        order = sorted(range(vocab), key=lambda i: (-logits[r, i].item(), i))[:p.logprobs]
        assert [t for t, _ in top] == order
        for t, v in top:
            assert abs(v - ref[r, t].item()) < 1e-4


@pytest.mark.gpu
def test_logprobs_through_the_engine_are_those_of_the_raw_distribution(tmp_path):
    from helpers import TINY, random_tokens, write_tiny
    from iian_b200 import EngineConfig, SamplingParams as SP
    from iian_b200.engine.engine import Engine
    d = write_tiny(str(tmp_path), "A")
    cfg, w = plain.load_folder(d)
    vocab = TINY["A"]["vocab_size"]
    prompt = random_tokens(vocab, 6, 9)
    eng = Engine(d, EngineConfig(dtype="float32", block_size=8, max_model_len=64, kv_cache_tokens=256))
    r = eng.submit(prompt, SP(temperature=0.0, max_tokens=6, ignore_eos=True, logprobs=3, repetition_penalty=1.5,
                              logit_bias={2: 3.0}))
    while not r.is_finished:
        eng.step()
    out = r.output_tokens
    assert len(r.logprobs) == len(out) == 6
    assert sum(len(c.logprobs) for c in r.outputs) == 6
    toks = list(prompt)
    for tok, (lp, top) in zip(out, r.logprobs):
        ref = torch.log_softmax(plain.forward(cfg, w, toks)[-1].double(), dim=-1)      # before bias and penalty
        assert abs(lp - ref[tok].item()) < 1e-3
        assert len(top) == 3 and top[0][0] == int(torch.argmax(ref)) and abs(top[0][1] - ref.max().item()) < 1e-3
        toks.append(tok)
