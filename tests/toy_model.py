"""A toy architecture that lives in the tests only: registered, built from a model folder and stepped through
the engine's own step function without a change to any file of the framework.

It has what Qwen3 does not: a mixer with a fixed-size state of its own per request (an exponential moving
average of its inputs, kept in a state slot), different mixers in different layers, a layer that runs twice
with a cache for each run, and a layer that reads the cache another layer filled.  A second layout has no
attention at all, so the model needs no pages.  The toy mixer computes with torch operations on the step's
device tensors only (never on the host lists), so its steps can be replayed from CUDA graphs; the attention,
norm and feed-forward parts beside it are the framework's.  ``plain_toy`` is the same model written out
separately in float64 on whole sequences.  A third layout has a feed-forward with routing (every token goes to 2 of
5 experts) and a position encoding that is no rotation (offsets added to Q and K), both defined here.  A fourth
arranges a layer's parts otherwise than the framework's block does: one norm feeds mixer and feed-forward side by
side, another layer has no feed-forward and norms its mixer's output (a slot of its own in ``LayerSpec.extra``).
"""
import math
import os

import torch

import plain_qwen3 as plain
from iian_b200.config.registry import Architecture, get_architecture, register_architecture, unregister_architecture
from iian_b200.config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from iian_b200.parts.base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, FeedForward, Mixer, PositionEncoding, StateNeed,
                                  register_block, register_feed_forward, register_mixer, register_position)
from iian_b200.weights.loader import TensorSpec

CFG = {"architectures": ["ToyForCausalLM"], "vocab_size": 97, "hidden_size": 64, "heads": 4, "kv_heads": 2, "head_dim": 16,
       "ffn": 96, "eps": 1e-5, "theta": 10000.0, "decay": 0.75, "max_position": 256, "layout": "mixed"}
CFG_EMA_ONLY = dict(CFG, layout="ema_only", vocab_size=61, hidden_size=48, ffn=80, decay=0.6)
# attention with a position encoding of the test's own (a table of offsets added to Q and K, not a rotation) and a
# feed-forward that routes every token to 2 of 5 small experts
# layers arranged otherwise than Qwen3's: one norm feeding mixer and feed-forward side by side, a layer without a
# feed-forward whose mixer output passes a norm of its own -- an arrangement defined here, beside the framework's own
CFG_PARALLEL = dict(CFG, layout="parallel", vocab_size=71, hidden_size=80, heads=5, kv_heads=5, head_dim=16, ffn=112, decay=0.7)
CFG_ROUTED = dict(CFG, layout="routed", vocab_size=83, hidden_size=72, heads=6, kv_heads=3, head_dim=24, ffn=40, experts=5, top_k=2,
                  max_position=160)


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


class ToyRoutedFF(FeedForward):
    """Routed experts: scores = x Wr^T in float32; the ``top_k`` best experts of a token get weights softmax(their
    scores); y = sum_e weight_e * W2_e relu(W1_e x).  Torch operations on whole tensors; it branches on nothing."""

    graph_safe = True

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.hidden, self.inter = int(spec["hidden_size"]), int(spec["intermediate_size"])
        self.n_experts, self.top_k = int(spec["experts"]), int(spec["top_k"])

    def tensors(self):
        return {"router": TensorSpec((self.n_experts, self.hidden)),
                "w1": TensorSpec((self.n_experts * self.inter, self.hidden)),
                "w2": TensorSpec((self.n_experts * self.hidden, self.inter))}

    def bind(self, tensors):
        self.router = tensors["router"].float()
        self.w1 = tensors["w1"].float().view(self.n_experts, self.inter, self.hidden)
        self.w2 = tensors["w2"].float().view(self.n_experts, self.hidden, self.inter)

    def forward(self, x, ctx):
        xf = x.float()
        scores = xf @ self.router.T                                          # [N, E], float32
        top, idx = torch.topk(scores, self.top_k, dim=-1)
        gate = torch.zeros_like(scores).scatter_(1, idx, torch.softmax(top, dim=-1))
        h = torch.relu(torch.einsum("nh,eih->nei", xf, self.w1))             # every expert on every token (it is a toy)
        y = torch.einsum("nei,ehi->neh", h, self.w2)
        return (gate[:, :, None] * y).sum(1).to(x.dtype)


class ToyOffsets(PositionEncoding):
    """A position encoding that is no rotation: a fixed table of offsets, indexed by the position, is added to every
    head of Q and of K before they are stored and used.  ``fused = False``: the attention mixer calls ``apply`` on the
    projected heads and hands the kernels unrotated heads."""

    fused = False
    dim = 0
    style = 0
    inv_freq = None

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        hd, n = int(spec["head_dim"]), int(spec["max_position"])
        pos = torch.arange(n, dtype=torch.float64)[:, None]
        j = torch.arange(hd, dtype=torch.float64)[None, :]
        self.table = (0.5 * torch.sin(pos * (j + 1) * 0.37)).to(torch.float32).to(device)    # [max_position, head_dim]

    def apply(self, qkv, num_heads, num_kv_heads, head_dim, ctx):
        n = qkv.shape[0]
        off = self.table[ctx.positions.long()]                               # [N, hd]
        heads = qkv.view(n, num_heads + 2 * num_kv_heads, head_dim)
        qk = heads[:, :num_heads + num_kv_heads]
        qk.copy_((qk.float() + off[:, None, :]).to(qkv.dtype))               # V is left alone


class ToyParallelBlock:
    """Another arrangement of a layer's parts than the framework's: ``x += mixer(norm(x)) + ffn(norm(x))`` with one
    norm feeding both (the feed-forward slot may be empty), and optionally a norm of the mixer's output before it is
    added (slot ``mixer_post_norm`` in ``LayerSpec.extra``).  The interface is what the model asks of any block."""

    def __init__(self, spec, dtype, device):
        self.dtype = dtype
        self.norm = NORMS.build(spec.mixer_norm, dtype, device)
        self.mixer = MIXERS.build(spec.mixer, dtype, device)
        self.ffn = FEED_FORWARDS.build(spec.feed_forward, dtype, device) if spec.feed_forward is not None else None
        post = spec.slot("mixer_post_norm")
        self.post = NORMS.build(post, dtype, device) if post is not None else None

    def parts(self):
        out = [("mixer_norm", self.norm), ("mixer", self.mixer)]
        if self.ffn is not None:
            out.append(("feed_forward", self.ffn))
        if self.post is not None:
            out.append(("mixer_post_norm", self.post))
        return tuple(out)

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, residual, delta, ctx, cache, writes_cache, select_rows):
        h = self.norm.forward(residual, delta, ctx)              # residual += delta; h = norm(residual)
        h_ffn = h.clone() if self.ffn is not None else None      # the mixer may reuse the norm's buffer
        y = self.mixer.forward(h, ctx, cache, writes_cache)
        if self.post is not None:
            y32 = y.float()
            y = (y32 * torch.rsqrt(y32.pow(2).mean(dim=-1, keepdim=True) + self.post.eps) * self.post.weight).to(self.dtype)
        if self.ffn is not None:
            y = (y.float() + self.ffn.forward(h_ffn, ctx).float()).to(self.dtype)
        if select_rows is not None:
            idx = select_rows.long()
            residual, y = residual.index_select(0, idx), y.index_select(0, idx)
        return residual, y


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
        elif c.get("layout") == "parallel":
            layers = (LayerSpec(mixer=attn, feed_forward=ffn, mixer_norm=norm, arrangement="toy_parallel"),
                      LayerSpec(mixer=ema, mixer_norm=norm, arrangement="toy_parallel", extra=(("mixer_post_norm", norm),)),
                      LayerSpec(attn, ffn, norm, norm))
            order = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(2, 2))
        elif c.get("layout") == "routed":
            offsets = PartSpec("toy_offsets", {"head_dim": c["head_dim"], "max_position": c["max_position"]})
            attn_off = PartSpec("attention", dict(attn.params, position=offsets))
            routed = PartSpec("toy_routed", {"hidden_size": H, "intermediate_size": c["ffn"], "experts": c["experts"], "top_k": c["top_k"]})
            layers = (LayerSpec(attn_off, routed, norm, norm), LayerSpec(attn_off, ffn, norm, norm), LayerSpec(attn, routed, norm, norm))
            order = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(2, 2))
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
    register_feed_forward("toy_routed")(ToyRoutedFF)
    register_position("toy_offsets")(ToyOffsets)
    register_block("toy_parallel")(ToyParallelBlock)
    register_architecture(ToyArch)
    return get_architecture("ToyForCausalLM")


def unregister_toy():
    unregister_architecture("ToyForCausalLM")
    MIXERS.unregister("toy_ema")
    FEED_FORWARDS.unregister("toy_routed")
    POSITIONS.unregister("toy_offsets")
    BLOCKS.pop("toy_parallel", None)


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

    def place(t, offsets):             # rotation, or the toy table of offsets added to every head
        if not offsets:
            return plain.rope_neox(t, pos, c["theta"], hd)
        j = torch.arange(hd, dtype=torch.float64)[None, :]
        table = (0.5 * torch.sin(pos.double()[:, None] * (j + 1) * 0.37)).float().double()
        return t + table[:, None, :]

    def attn_out(h, li, cache_id, writes, offsets=False):
        p = f"layer.{li}."
        q = place((h @ w[p + "mixer.q_proj.weight"].T).view(T, nh, hd), offsets)
        if writes:
            k = place((h @ w[p + "mixer.k_proj.weight"].T).view(T, nkv, hd), offsets)
            v = (h @ w[p + "mixer.v_proj.weight"].T).view(T, nkv, hd)
            kv[cache_id] = (k, v)
        k, v = kv[cache_id]
        a = plain.attention(q, k, v, 1 / math.sqrt(hd), None).reshape(T, nh * hd)
        return a @ w[p + "mixer.o_proj.weight"].T

    def attn_layer(x, li, cache_id, writes, offsets=False):
        h = plain.rms_norm(x, w[f"layer.{li}.mixer_norm.weight"], c["eps"])
        return x + attn_out(h, li, cache_id, writes, offsets)

    def ema_out(h, li):
        state = torch.zeros(c["hidden_size"], dtype=torch.float64)
        ys = []
        for t in range(T):
            state = c["decay"] * state + h[t]
            ys.append(w[f"layer.{li}.mixer.w"] @ state)
        return torch.stack(ys)

    def ema_layer(x, li):
        h = plain.rms_norm(x, w[f"layer.{li}.mixer_norm.weight"], c["eps"])
        return x + ema_out(h, li)

    def ffn(x, li):
        p = f"layer.{li}."
        h = plain.rms_norm(x, w[p + "feed_forward_norm.weight"], c["eps"])
        return x + plain.gated_mlp(h, w[p + "feed_forward.gate_proj.weight"], w[p + "feed_forward.up_proj.weight"],
                                   w[p + "feed_forward.down_proj.weight"])

    def routed(x, li):
        p = f"layer.{li}."
        h = plain.rms_norm(x, w[p + "feed_forward_norm.weight"], c["eps"])
        E, I, H = c["experts"], c["ffn"], c["hidden_size"]
        scores = h @ w[p + "feed_forward.router"].T
        w1 = w[p + "feed_forward.w1"].view(E, I, H)
        w2 = w[p + "feed_forward.w2"].view(E, H, I)
        out = torch.zeros_like(x)
        for t in range(T):
            top, idx = torch.topk(scores[t], c["top_k"])
            gate = torch.softmax(top, dim=-1)
            for g, e in zip(gate, idx):
                out[t] += g * (w2[e] @ torch.relu(w1[e] @ h[t]))
        return x + out

    if c.get("layout", "mixed") == "ema_only":
        x = ffn(ema_layer(x, 0), 0)
        x = ffn(ema_layer(x, 1), 1)
    elif c.get("layout") == "parallel":
        h = plain.rms_norm(x, w["layer.0.mixer_norm.weight"], c["eps"])        # one norm feeds mixer and feed-forward
        x = x + attn_out(h, 0, 0, True) + plain.gated_mlp(h, w["layer.0.feed_forward.gate_proj.weight"],
                                                        w["layer.0.feed_forward.up_proj.weight"], w["layer.0.feed_forward.down_proj.weight"])
        h = plain.rms_norm(x, w["layer.1.mixer_norm.weight"], c["eps"])        # no feed-forward; the mixer's output is normed
        x = x + plain.rms_norm(ema_out(h, 1), w["layer.1.mixer_post_norm.weight"], c["eps"])
        x = ffn(attn_layer(x, 2, 2, True), 2)
    elif c.get("layout") == "routed":
        x = routed(attn_layer(x, 0, 0, True, offsets=True), 0)
        x = ffn(attn_layer(x, 1, 1, True, offsets=True), 1)
        x = routed(attn_layer(x, 2, 2, True), 2)
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
