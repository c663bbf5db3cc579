"""A plain, slow implementation of Qwen3 dense: whole sequences, no cache, one function per part.

It is written from the reference's formulas (each function cites file:line under the reference's
tree) and shares no code with ``iian_b200``: it reads ``config.json`` and the safetensors file itself
and computes with elementary torch tensor operations on the CPU, in float64 by default so that
it can serve as the oracle for both the 32-bit and the bfloat16 path.

``tests/golden/`` holds logits that the reference's own model code produced for a tiny random model;
``test_plain_vs_golden`` checks this file against them, so it rests on the reference's code as well
as on its formulas.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


# ---- files ---------------------------------------------------------------------------------------
def read_safetensors(path: str, keep32: bool = False) -> Dict[str, torch.Tensor]:
    """Every tensor of a safetensors file as float64 (integers as int64).  ``keep32``: tensors stored in 16 or 32
    bits stay float32 (the same values in half the memory; for models of several GB)."""
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen).decode("utf-8"))
        base = 8 + hlen
    data = np.memmap(path, dtype=np.uint8, mode="r", offset=base) if os.path.getsize(path) > base else np.zeros(0, np.uint8)
    wide = (lambda t: t) if keep32 else (lambda t: t.double())
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = data[b:e]
        shape = info["shape"]
        tag = info["dtype"]
        if tag == "F32":
            t = wide(torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy()))
        elif tag == "F16":
            t = wide(torch.from_numpy(np.frombuffer(raw, dtype="<f2").copy()).float())
        elif tag == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            t = wide(torch.from_numpy(u.view(np.float32).copy()))
        elif tag == "F64":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<f8").copy())
        elif tag in ("I32", "I64"):
            t = torch.from_numpy(np.frombuffer(raw, dtype="<i4" if tag == "I32" else "<i8").copy()).long()
        else:
            raise ValueError(f"{path}: dtype {tag} of '{name}' is not handled")
        out[name] = t.reshape(shape)
    return out


def load_folder(model_dir: str, keep32: bool = False):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"), keep32)


class _CastOnUse:
    """The weights by name, widened to the computing dtype each time one is used (nothing is kept)."""

    def __init__(self, w: Dict[str, torch.Tensor], dtype):
        self.w, self.dtype = w, dtype

    def __getitem__(self, k):
        v = self.w[k]
        return v.to(self.dtype) if v.is_floating_point() else v

    def get(self, k, default=None):
        return self[k] if k in self.w else default

    def __contains__(self, k):
        return k in self.w


# ---- parts ---------------------------------------------------------------------------------------
def embedding(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """x0[t] = E[token_t]  (src/iian/graph.cpp:39-46)."""
    return table[torch.as_tensor(list(tokens), dtype=torch.long)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps), then * weight; no 1 + w, no bias  (src/iian/graph.cpp:105-114)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def rope_neox(x: torch.Tensor, positions: torch.Tensor, base: float, n_rot: int) -> torch.Tensor:
    """NEOX rotation of x [T, heads, hd]: for j < n_rot/2, theta = pos * base^(-2j/n_rot);
    (x_j, x_{j+n_rot/2}) <- (x_j cos - x_{j+n_rot/2} sin, x_j sin + x_{j+n_rot/2} cos)
    (third_party/ggml/src/ggml-cpu/ops.cpp:5958-5990, 6063-6079; src/iian/arch/qwen3.cpp:106).
    The per-pair factor base^(-2j/n_rot) is rounded to float32 as an inference engine holds it."""
    half = n_rot // 2
    j = torch.arange(half, dtype=torch.float64)
    inv_freq = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * j / n_rot).float().double()
    theta = (positions.float()[:, None] * inv_freq.float()[None, :]).double()    # the product is float32, too
    cos, sin = torch.cos(theta)[:, None, :], torch.sin(theta)[:, None, :]
    x0, x1 = x[..., :half], x[..., half:n_rot]
    out = x.clone()
    out[..., :half] = x0 * cos - x1 * sin
    out[..., half:n_rot] = x0 * sin + x1 * cos
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int]) -> torch.Tensor:
    """q [T, nh, hd], k/v [T, nkv, hd] of one whole sequence.  Head h uses KV head h // (nh/nkv);
    s = q.k * scale; key j visible iff j <= t and (no window or t - j < window); softmax; sum p v
    (src/iian/paged_attn.cpp:112-145, window test :124; src/iian/arch/qwen3.cpp:72, 89)."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    out = torch.zeros_like(q)
    t_idx = torch.arange(T)
    visible = t_idx[None, :] <= t_idx[:, None]
    if window:
        visible &= (t_idx[:, None] - t_idx[None, :]) < window
    for h in range(nh):
        kh = h // g
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, kh, :]
    return out


def silu(z: torch.Tensor) -> torch.Tensor:
    """z / (1 + exp(-z))  (third_party/ggml/src/ggml-cpu/vec.h:1046-1048)."""
    return z / (1.0 + torch.exp(-z))


def gated_mlp(h: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """Wdown (silu(Wgate h) * (Wup h))  (src/iian/graph.cpp:116-163, :135; src/iian/arch/qwen3.cpp:97)."""
    return (silu(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


# ---- whole model ---------------------------------------------------------------------------------
def layer_windows(cfg: dict) -> List[Optional[int]]:
    n = cfg["num_hidden_layers"]
    win = cfg.get("sliding_window")
    types = cfg.get("layer_types")
    if types is None:
        if cfg.get("use_sliding_window") and win:
            first = cfg.get("max_window_layers", n)
            types = ["sliding_attention" if i >= first else "full_attention" for i in range(n)]
        else:
            types = ["full_attention"] * n
    return [win if t == "sliding_attention" else None for t in types]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], dtype=torch.float64,
            return_hidden: bool = False) -> torch.Tensor:
    """Logits [T, vocab] at every position of one sequence (src/iian/arch/qwen3.cpp:61-104)."""
    W = _CastOnUse(w, dtype)
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads", nh)
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    eps = cfg.get("rms_norm_eps", 1e-6)
    base = cfg.get("rope_theta", 10000.0)
    T = len(tokens)
    pos = torch.arange(T)
    windows = layer_windows(cfg)
    x = embedding(w["model.embed_tokens.weight"], tokens).to(dtype)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = rms_norm(x, W[p + "input_layernorm.weight"], eps)                         # qwen3.cpp:77
        q = h @ W[p + "self_attn.q_proj.weight"].T                                    # qwen3.cpp:80
        k = h @ W[p + "self_attn.k_proj.weight"].T
        v = h @ W[p + "self_attn.v_proj.weight"].T
        for n_, t_ in (("q", q), ("k", k), ("v", v)):
            b = W.get(p + f"self_attn.{n_}_proj.bias")
            if b is not None:
                t_ += b
        q = q.view(T, nh, hd)
        k = k.view(T, nkv, hd)
        v = v.view(T, nkv, hd)
        q = rms_norm(q, W[p + "self_attn.q_norm.weight"], eps)                        # qwen3.cpp:82
        k = rms_norm(k, W[p + "self_attn.k_norm.weight"], eps)                        # qwen3.cpp:85
        q = rope_neox(q, pos, base, hd).to(dtype)                                      # qwen3.cpp:84
        k = rope_neox(k, pos, base, hd).to(dtype)                                      # qwen3.cpp:87
        a = attention(q, k, v, 1.0 / math.sqrt(hd), windows[i]).reshape(T, nh * hd)    # qwen3.cpp:72, 89
        o = a @ W[p + "self_attn.o_proj.weight"].T
        if p + "self_attn.o_proj.bias" in W:
            o = o + W[p + "self_attn.o_proj.bias"]
        x = x + o                                                                      # qwen3.cpp:92
        h2 = rms_norm(x, W[p + "post_attention_layernorm.weight"], eps)               # qwen3.cpp:95
        x = x + gated_mlp(h2, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"],
                          W[p + "mlp.down_proj.weight"])                              # qwen3.cpp:97-99
    xn = rms_norm(x, W["model.norm.weight"], eps)                                     # qwen3.cpp:103
    if return_hidden:
        return xn
    return head(w, xn, dtype)


def head(w: Dict[str, torch.Tensor], xn: torch.Tensor, dtype=torch.float64) -> torch.Tensor:
    """Logits of normalised rows: the output matrix if the file has one, else the embedding (qwen3.cpp:26-27, 103)."""
    w_out = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return xn.to(dtype) @ w_out.to(dtype).T


# ---- sampling ------------------------------------------------------------------------------------
def argmax(logits: torch.Tensor) -> int:
    """First index of the maximum: ties go to the lowest id  (src/iian/vec_math.h:78-82)."""
    mx = logits.max()
    return int((logits == mx).nonzero()[0, 0])


def candidate_probs(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0,
                    min_p: float = 0.0) -> torch.Tensor:
    """Unnormalised probabilities exp(z - max) of the kept candidates (0 elsewhere), z = logits / T:
    min_p keeps z >= max + log(min_p); top_k the k largest by (value desc, id asc) if k < count; top_p
    the shortest prefix in that order whose share of the kept mass reaches top_p
    (src/iian/sampler.cpp:115-163)."""
    inv_t = np.float32(1.0) / np.float32(temperature)
    z = (logits.float() * float(inv_t)).double()          # the scaling is a float32 product
    V = z.numel()
    keep = torch.ones(V, dtype=torch.bool)
    mx = z.max()
    if min_p > 0:
        keep &= z.float() >= (mx.float() + np.float32(math.log(np.float32(min_p))))
    order = sorted(range(V), key=lambda i: (-float(z[i]), i))
    order = [i for i in order if keep[i]]
    if 0 < top_k < len(order):
        order = order[:top_k]
    e = torch.exp(z - mx)
    if top_p < 1.0 and len(order) > 1:
        total = sum(float(e[i]) for i in order)
        cum, kept = 0.0, []
        for i in order:
            cum += float(e[i])
            kept.append(i)
            if cum >= top_p * total:
                break
        order = kept
    out = torch.zeros(V, dtype=torch.float64)
    for i in order:
        out[i] = e[i]
    return out


def sample_from(probs: torch.Tensor, u: float) -> int:
    """Inverse CDF in vocabulary order: the first id whose running mass exceeds u * total
    (the walk of src/iian/sampler.cpp:165-171, in id order)."""
    total = float(probs.sum())
    r = u * total
    run = 0.0
    last = 0
    for i in range(probs.numel()):
        p = float(probs[i])
        if p > 0:
            last = i
            run += p
            if run > r:
                return i
    return last


def process_logits(logits: torch.Tensor, prompt: Sequence[int], output: Sequence[int], *, allowed=(), bias=None,
                   bad_words=(), banned=(), presence=0.0, frequency=0.0, repetition=1.0, last_n=-1) -> torch.Tensor:
    """The logits processors on one row, dense and in the reference's order (src/iian/sampler.cpp:72-109): allowed
    ids (:72-76), logit bias (:77), bad words (:78-88), ids that may not be produced yet (the caller's EOS mask while
    min_tokens holds, :89-91), then the penalties over the counts of the last ``last_n`` output tokens, the
    repetition penalty reaching prompt tokens too (:93-109)."""
    l = logits.clone().double()
    n_vocab = l.numel()
    if len(allowed):
        keep = torch.full_like(l, float("-inf"))
        for t in allowed:
            if 0 <= t < n_vocab:
                keep[t] = l[t]
        l = keep
    for t, b in (bias or {}).items():
        l[t] += b
    n_out = len(output)
    for bw in bad_words:
        if not len(bw):
            continue
        pre = len(bw) - 1
        if n_out < pre:
            continue
        if all(output[n_out - pre + i] == bw[i] for i in range(pre)) and 0 <= bw[-1] < n_vocab:
            l[bw[-1]] = float("-inf")
    for t in banned:
        l[t] = float("-inf")
    if repetition != 1.0 or presence != 0.0 or frequency != 0.0:
        counts: Dict[int, int] = {}
        start = 0 if last_n < 0 else max(0, n_out - last_n)
        for t in output[start:]:
            counts[t] = counts.get(t, 0) + 1
        if repetition != 1.0:
            for t in prompt:
                counts.setdefault(t, 0)
        for t, c in counts.items():
            if t < 0 or t >= n_vocab:
                continue
            if repetition != 1.0:
                l[t] = l[t] / repetition if l[t] > 0 else l[t] * repetition
            if c > 0:
                l[t] -= frequency * c + presence
    return l
