"""A toy architecture defined entirely in this test, registered, built from a model folder and stepped
through the engine's own step function -- without a change to any file of the framework.

It has what Qwen3 does not: a mixer with a fixed-size state of its own per request (an exponential
moving average of its inputs, kept in a state slot), different mixers in different layers, a layer that
runs twice with a cache for each run, and a layer that reads the cache another layer filled.  The toy
parts compute with torch operations (they are test code); the attention, norm and feed-forward parts
beside them are the framework's.  The plain model at the bottom is written out separately in float64.
"""
import json
import math
import os

import pytest
import torch

import plain_qwen3 as plain
from helpers import first_bad, random_tokens, replay_and_collect, trace_mixed, trace_portions, trace_tail, trace_whole
from iian_b200.config.registry import Architecture, get_architecture, register_architecture, unregister_architecture
from iian_b200.config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from iian_b200.parts.base import MIXERS, Mixer, StateNeed, register_mixer
from iian_b200.weights.loader import TensorSpec

pytestmark = pytest.mark.gpu

CFG = {"architectures": ["ToyForCausalLM"], "vocab_size": 97, "hidden_size": 64, "heads": 4, "kv_heads": 2, "head_dim": 16,
       "ffn": 96, "eps": 1e-5, "theta": 10000.0, "decay": 0.75, "max_position": 256}


class ToyEma(Mixer):
    """state_t = decay * state_{t-1} + x_t;  y_t = W state_t.  The state lives in the request's slot."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.decay = float(spec["decay"])
        self.w = None

    def tensors(self):
        return {"w": TensorSpec((self.hidden, self.hidden))}

    def bind(self, tensors):
        self.w = tensors["w"].float()

    def cache_need(self):
        return StateNeed((self.hidden,), torch.float32)

    def forward(self, x, ctx, cache, writes_cache):
        out = torch.empty_like(x)
        for start, n, slot in zip(ctx.h_q_start, ctx.h_q_len, ctx.h_state_slots):
            state = cache.state[slot]
            for t in range(start, start + n):               # a portion continues the state the last one left
                state = self.decay * state + x[t].float()
                out[t] = (self.w @ state).to(x.dtype)
            cache.state[slot] = state
        return out


class ToyArch(Architecture):
    name = "ToyForCausalLM"

    def load_config(self, raw):
        return dict(raw)

    def config_to_dict(self, c):
        return dict(c)

    def build_spec(self, c):
        H = c["hidden_size"]
        norm = PartSpec("rms_norm", {"size": H, "eps": c["eps"]})
        attn = PartSpec("attention", {"hidden_size": H, "num_heads": c["heads"], "num_kv_heads": c["kv_heads"],
                                      "head_dim": c["head_dim"], "scale": 1 / math.sqrt(c["head_dim"]), "qk_norm": False,
                                      "window": None,
                                      "position": PartSpec("rotary", {"dim": c["head_dim"], "base": c["theta"], "style": "neox"})})
        ema = PartSpec("toy_ema", {"hidden_size": H, "decay": c["decay"]})
        ffn = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": c["ffn"]})
        layers = (LayerSpec(attn, ffn, norm, norm), LayerSpec(ema, ffn, norm, norm), LayerSpec(attn, ffn, norm, norm))
        # layer 0 runs twice (caches 0 and 2); layer 2 reads the cache layer 0 filled on its first run
        order = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(2, 0, writes_cache=False), LayerCall(0, 2))
        return ModelSpec(H, c["vocab_size"], c["max_position"], PartSpec("token_embedding", {"vocab_size": c["vocab_size"], "hidden_size": H}),
                         layers, order, norm, PartSpec("lm_head", {"hidden_size": H, "vocab_size": c["vocab_size"], "tied": True}))

    def tensor_name(self, scope, local):
        return ".".join(str(s) for s in scope) + "." + local


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    register_mixer("toy_ema")(ToyEma)
    register_architecture(ToyArch)
    from iian_b200.weights.random_init import write_model_folder
    d = str(tmp_path_factory.mktemp("toy"))
    arch = get_architecture("ToyForCausalLM")
    write_model_folder(d, arch, dict(CFG), seed=9, store_dtype=torch.bfloat16, std=0.08)
    yield d
    unregister_architecture("ToyForCausalLM")
    MIXERS.unregister("toy_ema")


def plain_toy(d, tokens):
    """The toy model on one whole sequence, in float64, written out without the framework."""
    w = plain.read_safetensors(os.path.join(d, "model.safetensors"))
    c = CFG
    T, nh, nkv, hd = len(tokens), c["heads"], c["kv_heads"], c["head_dim"]
    pos = torch.arange(T)
    x = w["embedding.weight"][torch.tensor(tokens)]
    kv = {}

    def attn_layer(x, li, cache_id, writes):
        p = f"layer.{li}."
        h = plain.rms_norm(x, w[p + "mixer_norm.weight"], c["eps"])
        q = plain.rope_neox((h @ w[p + "mixer.q_proj.weight"].T).view(T, nh, hd), pos, c["theta"], hd)
        if writes:
            k = plain.rope_neox((h @ w[p + "mixer.k_proj.weight"].T).view(T, nkv, hd), pos, c["theta"], hd)
            v = (h @ w[p + "mixer.v_proj.weight"].T).view(T, nkv, hd)
            kv[cache_id] = (k, v)
        k, v = kv[cache_id]
        a = plain.attention(q, k, v, 1 / math.sqrt(hd), None).reshape(T, nh * hd)
        return x + a @ w[p + "mixer.o_proj.weight"].T

    def ema_layer(x, li):
        p = f"layer.{li}."
        h = plain.rms_norm(x, w[p + "mixer_norm.weight"], c["eps"])
        state = torch.zeros(c["hidden_size"], dtype=torch.float64)
        ys = []
        for t in range(T):
            state = c["decay"] * state + h[t]
            ys.append(w[p + "mixer.w"] @ state)
        return x + torch.stack(ys)

    def ffn(x, li):
        p = f"layer.{li}."
        h = plain.rms_norm(x, w[p + "feed_forward_norm.weight"], c["eps"])
        return x + plain.gated_mlp(h, w[p + "feed_forward.gate_proj.weight"], w[p + "feed_forward.up_proj.weight"],
                                   w[p + "feed_forward.down_proj.weight"])

    x = ffn(attn_layer(x, 0, 0, True), 0)
    x = ffn(ema_layer(x, 1), 1)
    x = ffn(attn_layer(x, 2, 0, False), 2)
    x = ffn(attn_layer(x, 0, 2, True), 0)
    return plain.rms_norm(x, w["final_norm.weight"], c["eps"]) @ w["embedding.weight"].T


def test_toy_is_built_from_registered_parts(toy):
    from iian_b200.engine.model import Model
    m = Model.from_folder(toy, "float32", "cuda:0")
    assert m.arch.name == "ToyForCausalLM"
    assert [type(b.mixer).__name__ for b in m.blocks] == ["Attention", "ToyEma", "Attention"]
    needs = m.cache_needs()
    assert sorted(needs) == [0, 1, 2] and isinstance(needs[1], StateNeed) and needs[0] == needs[2]
    with open(os.path.join(toy, "config.json")) as f:
        assert json.load(f)["architectures"] == ["ToyForCausalLM"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_toy_steps_like_its_plain_model(toy, dtype, mode):
    from iian_b200.engine.replay import TraceReplayer
    reqs = {f"r{i}": random_tokens(CFG["vocab_size"], n, 70 + i) for i, n in enumerate([3, 40, 21, 64, 9, 33])}
    want = {rid: plain_toy(toy, toks) for rid, toks in reqs.items()}
    steps = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions}.get(mode)
    steps = steps(reqs) if steps else trace_mixed(reqs, 192, seed=4, max_live=3)
    rp = TraceReplayer.from_folder(toy, dtype, 192, block_size=8, max_requests=3)     # 3 slots: they are used again
    got = replay_and_collect(rp, steps)
    scale = max(v.abs().max().item() for v in want.values())
    tol = 3e-5 * max(scale, 1.0) if dtype == "float32" else 2.5e-2 * scale
    bad = first_bad(got, want, tol)
    assert bad is None, f"first wrong logits at request {bad[0]} position {bad[1]} (err {bad[2]:.3g}, tol {tol:.3g})"
    assert len(got) == sum(len(t) for t in reqs.values())
    assert rp.runner.manager.slots.num_free == 3 and all(p.num_free == p.num_blocks for p in rp.runner.manager.pools)
