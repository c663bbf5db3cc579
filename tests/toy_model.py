"""A toy architecture that lives in the tests only: registered, built from a model folder and stepped through
the engine's own step function without a change to any file of the framework.

It has what Qwen3 does not: a mixer with a fixed-size state of its own per request (an exponential moving
average of its inputs, kept in a state slot), different mixers in different layers, a layer that runs twice
with a cache for each run, and a layer that reads the cache another layer filled.  A second layout has no
attention at all, so the model needs no pages.  The toy mixer computes with torch operations on the step's
device tensors only (never on the host lists), so its steps can be replayed from CUDA graphs; the attention,
norm and feed-forward parts beside it are the framework's.  ``plain_toy`` is the same model written out
separately in float64 on whole sequences.
"""
import math
import os

import torch

import plain_qwen3 as plain
from iian_b200.config.registry import Architecture, get_architecture, register_architecture, unregister_architecture
from iian_b200.config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from iian_b200.parts.base import MIXERS, Mixer, StateNeed, register_mixer
from iian_b200.weights.loader import TensorSpec

CFG = {"architectures": ["ToyForCausalLM"], "vocab_size": 97, "hidden_size": 64, "heads": 4, "kv_heads": 2, "head_dim": 16,
       "ffn": 96, "eps": 1e-5, "theta": 10000.0, "decay": 0.75, "max_position": 256, "layout": "mixed"}
CFG_EMA_ONLY = dict(CFG, layout="ema_only", vocab_size=61, hidden_size=48, ffn=80, decay=0.6)


class ToyEma(Mixer):
    """state_t = decay * state_{t-1} + x_t;  y_t = W state_t.  The state lives in the request's slot.

    For the tokens of one step: state_t = decay^(j+1) * state_before + sum_{i <= t, same request} decay^(t-i) x_i
    with j the token's place in its portion.  Padding rows (sequence -1 or slot -1) change nothing."""

    graph_safe = True

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
        n = x.shape[0]
        dev = x.device
        seq = ctx.seq_of_token.long()
        seq0 = seq.clamp(min=0)
        cu = ctx.cu_q.long()
        slots = ctx.state_slots.long()
        slot_t = slots[seq0]
        valid_t = (seq >= 0) & (slot_t >= 0)
        idx = torch.arange(n, device=dev)
        place = idx - cu[seq0]                                              # the token's place in its portion
        same = (seq[:, None] == seq[None, :]) & (idx[None, :] <= idx[:, None]) & valid_t[:, None]
        power = (idx[:, None] - idx[None, :]).clamp(min=0).to(torch.float32)
        mix = torch.pow(self.decay, power) * same.to(torch.float32)
        before = cache.state[slot_t.clamp(min=0)]                           # [N, H]
        carry = torch.pow(self.decay, (place + 1).clamp(min=0).to(torch.float32))
        states = (mix @ x.float() + carry[:, None] * before) * valid_t[:, None].to(torch.float32)
        out = (states @ self.w.T).to(x.dtype)
        # the state after each request's last token of this step goes back to its slot; written as an atomic
        # add of (new - old) so that padding sequences (which add zero to slot 0) need no branch
        n_seq = slots.shape[0]
        last = (cu[1:n_seq + 1] - 1).clamp(min=0)
        valid_s = slots >= 0
        old = cache.state[slots.clamp(min=0)]
        delta = (states[last] - old) * valid_s[:, None].to(torch.float32)
        cache.state.index_put_((slots.clamp(min=0),), delta, accumulate=True)
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
        if c.get("layout", "mixed") == "ema_only":
            layers = (LayerSpec(ema, ffn, norm, norm), LayerSpec(ema, ffn, norm, norm))
            order = (LayerCall(0, 0), LayerCall(1, 1))
        else:
            layers = (LayerSpec(attn, ffn, norm, norm), LayerSpec(ema, ffn, norm, norm), LayerSpec(attn, ffn, norm, norm))
            # layer 0 runs twice (caches 0 and 2); layer 2 reads the cache layer 0 filled on its first run
            order = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(2, 0, writes_cache=False), LayerCall(0, 2))
        return ModelSpec(H, c["vocab_size"], c["max_position"], PartSpec("token_embedding", {"vocab_size": c["vocab_size"], "hidden_size": H}),
                         layers, order, norm, PartSpec("lm_head", {"hidden_size": H, "vocab_size": c["vocab_size"], "tied": True}))

    def tensor_name(self, scope, local):
        return ".".join(str(s) for s in scope) + "." + local


def register_toy():
    register_mixer("toy_ema")(ToyEma)
    register_architecture(ToyArch)
    return get_architecture("ToyForCausalLM")


def unregister_toy():
    unregister_architecture("ToyForCausalLM")
    MIXERS.unregister("toy_ema")


def write_toy(d, cfg, seed=9):
    from iian_b200.weights.random_init import write_model_folder
    write_model_folder(d, get_architecture("ToyForCausalLM"), dict(cfg), seed=seed, store_dtype=torch.bfloat16, std=0.08)
    return d


def plain_toy(d, tokens, c=CFG):
    """The toy model on one whole sequence, in float64, written out without the framework."""
    w = plain.read_safetensors(os.path.join(d, "model.safetensors"))
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

    if c.get("layout", "mixed") == "ema_only":
        x = ffn(ema_layer(x, 0), 0)
        x = ffn(ema_layer(x, 1), 1)
    else:
        x = ffn(attn_layer(x, 0, 0, True), 0)
        x = ffn(ema_layer(x, 1), 1)
        x = ffn(attn_layer(x, 2, 0, False), 2)
        x = ffn(attn_layer(x, 0, 2, True), 0)
    return plain.rms_norm(x, w["final_norm.weight"], c["eps"]) @ w["embedding.weight"].T


def plain_toy_greedy(d, prompt, n, c=CFG):
    toks, margins = list(prompt), []
    for _ in range(n):
        row = plain_toy(d, toks, c)[-1]
        top = torch.topk(row, 2).values
        margins.append((top[0] - top[1]).item())
        toks.append(plain.argmax(row))
    return toks[len(prompt):], margins
