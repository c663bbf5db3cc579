"""Whole-model logits at the layer sizes of the Qwen3-8B shape (hidden 4096, 32 query heads on 8 KV heads of 128,
feed-forward 12288, vocabulary 151936), with 2 of its 36 layers so that the plain implementation can follow on
the CPU: reductions over 4096 and 12288 terms, a head of 151936 columns, tiles of 256 x 256 in several waves --
what the tiny configurations cannot show.

The 32-bit engine is held to 1e-4 (max abs) of the float64 plain implementation under every way of cutting the
work.  The bfloat16 engine is held to the plain implementation on the same traces, and to the (then checked)
32-bit engine on what would be slow to follow on the CPU: a step of more than 1024 rows, decoding from captured
graphs for 40 steps, and decode batches of 64, 16, 8 and 1.
"""
import pytest
import torch

import plain_qwen3 as plain
from helpers import first_bad, max_error, random_tokens, replay_and_collect, trace_mixed, trace_portions, trace_tail, trace_whole

pytestmark = pytest.mark.gpu

LAYERS_OF_SHAPE = 36
SIZES = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=2, num_attention_heads=32,
             num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=40960,
             tie_word_embeddings=False)
LENGTHS = [96, 40, 70, 33]
TOL32 = 1e-4
TOL16_REL = 2.5e-2


@pytest.fixture(scope="module")
def big(tmp_path_factory):
    """The model folder (drawn on the GPU: the same bits as on the CPU, much faster), the plain implementation's
    view of it, the requests and their plain logits."""
    from iian_b200.config.registry import get_architecture
    from iian_b200.models.qwen3 import qwen3_config_from_dict
    from iian_b200.weights.random_init import write_model_folder
    d = str(tmp_path_factory.mktemp("sizes8b"))
    write_model_folder(d, get_architecture("Qwen3ForCausalLM"), qwen3_config_from_dict(SIZES), seed=21,
                       store_dtype=torch.bfloat16, device="cuda:0")
    cfg, w = plain.load_folder(d, keep32=True)
    reqs = {f"r{i}": random_tokens(SIZES["vocab_size"], n, 300 + i) for i, n in enumerate(LENGTHS)}
    want = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    return d, cfg, w, reqs, want


@pytest.fixture(scope="module")
def models(big):
    from iian_b200.engine.model import Model
    d = big[0]
    return {dt: Model.from_folder(d, dt, "cuda:0") for dt in ("float32", "bfloat16")}


def traces(reqs):
    return {"whole": trace_whole(reqs), "tail": trace_tail(reqs), "portions": trace_portions(reqs),
            "mixed": trace_mixed(reqs, 256, seed=8)}


@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_32_bit_engine_against_the_plain_implementation(big, models, mode):
    from iian_b200.engine.replay import TraceReplayer
    _, _, _, reqs, want = big
    rp = TraceReplayer(models["float32"], 256, 16, 4)
    got = replay_and_collect(rp, traces(reqs)[mode])
    assert len(got) == sum(LENGTHS)
    worst, where = max_error(got, want)
    print(f"[8B sizes, 2 of {LAYERS_OF_SHAPE} layers, float32, {mode}] max abs err {worst:.3g} at {where}")
    bad = first_bad(got, want, TOL32)
    assert bad is None, f"first wrong logits at request {bad[0]} position {bad[1]} (err {bad[2]:.3g})"


@pytest.mark.parametrize("min_tiles", [0, 300])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_bfloat16_engine_against_the_plain_implementation(big, models, monkeypatch, mode, min_tiles):
    from iian_b200.engine.replay import TraceReplayer
    from iian_b200.ops import cuda_backend
    monkeypatch.setattr(cuda_backend.CudaKernels, "TCGEN05_MIN_TILES", min_tiles)
    _, _, _, reqs, want = big
    rp = TraceReplayer(models["bfloat16"], 256, 16, 4)
    got = replay_and_collect(rp, traces(reqs)[mode])
    rp.runner.check_device_status()
    tol = TOL16_REL * max(v.abs().max().item() for v in want.values())
    worst, where = max_error(got, want)
    print(f"[8B sizes, bfloat16, {mode}, min tiles {min_tiles}] max abs err {worst:.3g} at {where}, tol {tol:.3g}")
    bad = first_bad(got, want, tol)
    assert bad is None, f"first wrong logits at request {bad[0]} position {bad[1]} (err {bad[2]:.3g}, tol {tol:.3g})"


def _both(models, steps_of, max_tokens, max_requests, graphs):
    """The same steps through the 32-bit engine (eagerly) and the bfloat16 engine; rows of logits by (request, position)."""
    from iian_b200.engine.replay import TraceReplayer
    out = []
    for dt in ("float32", "bfloat16"):
        rp = TraceReplayer(models[dt], max_tokens, 16, max_requests)
        rp.runner.cuda_graphs = graphs and dt == "bfloat16"
        out.append((replay_and_collect(rp, steps_of), rp))
    return out


@pytest.mark.parametrize("min_tiles", [0, 300])
def test_a_step_of_more_than_1024_rows(big, models, monkeypatch, min_tiles):
    """One prompt of 1100 tokens in one step: the tcgen05 product on pairs of SMs with its SwiGLU epilogue (and,
    with the threshold at 0, with the folded norms) and tcgen05 attention over 9 key tiles; then 3 single tokens."""
    from iian_b200.ops import cuda_backend
    monkeypatch.setattr(cuda_backend.CudaKernels, "TCGEN05_MIN_TILES", min_tiles)
    toks = random_tokens(SIZES["vocab_size"], 1103, 77)
    steps = [{"step": 0, "entries": [{"id": "p", "tokens": toks[:1100], "want": [0, 127, 128, 511, 1023, 1024, 1099]}], "end": []}]
    for i in range(3):
        steps.append({"step": 1 + i, "entries": [{"id": "p", "tokens": [toks[1100 + i]], "want": [0]}], "end": ["p"] if i == 2 else []})
    before = dict(cuda_backend.LAUNCHES_BY_ENTRY)
    (a, _), (b, rp) = _both(models, steps, 1152, 2, graphs=False)
    rp.runner.check_device_status()
    seen = {k for k, v in rp.runner.launches_by_entry().items() if v > before.get(k, 0)}
    assert {"gemm_tcgen05", "attention_tc"} <= seen
    assert ("library_gemm" in seen) == (min_tiles > 0)
    scale = max(v.abs().max().item() for v in a.values())
    worst = max((a[k] - b[k]).abs().max().item() for k in a)
    print(f"[8B sizes, 1100 rows, min tiles {min_tiles}] bfloat16 against float32: {worst:.3g} (scale {scale:.3g})")
    assert len(a) == 10 and worst <= TOL16_REL * scale


def test_decoding_from_graphs_at_batches_of_64_16_8_and_1(big, models):
    """64 requests with short prompts; decode steps replayed from graphs while requests end: batches of 64, 16, 8
    (for 40 steps) and 1.  Rows 9..127 of the products, the key splits chosen for many sequences, padded batches."""
    v = SIZES["vocab_size"]
    ids = [f"q{i}" for i in range(64)]
    prompts = {r: random_tokens(v, 4 + (5 * i) % 19, 500 + i) for i, r in enumerate(ids)}
    nxt = {r: random_tokens(v, 64, 700 + i) for i, r in enumerate(ids)}
    steps, n = [], 0
    for i in range(0, 64, 16):                       # prompts, sixteen requests to a step
        steps.append({"step": n, "entries": [{"id": r, "tokens": prompts[r], "want": [len(prompts[r]) - 1]} for r in ids[i:i + 16]], "end": []})
        n += 1
    used = {r: 0 for r in ids}

    def decode(live, count, end=()):
        nonlocal n
        for c in range(count):
            ents = []
            for r in live:
                ents.append({"id": r, "tokens": [nxt[r][used[r]]], "want": [0]})
                used[r] += 1
            steps.append({"step": n, "entries": ents, "end": list(end) if c == count - 1 else []})
            n += 1

    decode(ids, 3, end=ids[16:])
    decode(ids[:16], 3, end=ids[8:16])
    decode(ids[:8], 40, end=ids[1:8])
    decode(ids[:1], 3, end=ids[:1])
    (a, _), (b, rp) = _both(models, steps, 64 * 80, 64, graphs=True)
    assert rp.runner.num_graphs >= 4, f"{rp.runner.num_graphs} graphs captured for batches of 64, 16, 8 and 1"
    scale = max(v_.abs().max().item() for v_ in a.values())
    worst, where = 0.0, None
    for k in a:
        e = (a[k] - b[k]).abs().max().item()
        if not e <= worst:
            worst, where = e, k
    print(f"[8B sizes, graphs, batches 64/16/8/1] bfloat16 against float32: {worst:.3g} at {where} (scale {scale:.3g})")
    assert len(a) == 64 + 64 * 3 + 16 * 3 + 8 * 40 + 3 and worst <= TOL16_REL * scale
