"""The attention mixer: projections, optional per-head RMSNorm of Q and K, position encoding, paged
cache write, attention over the cache, output projection.

Formulas in the reference's order (src/iian/arch/qwen3.cpp:80-89, src/iian/graph.cpp:215-244,
:308-354): ``q = Wq h``, ``k = Wk h``, ``v = Wv h`` (biases only where the file has them); Q and K
normalised over the head axis with one weight per projection; rotation; K and V stored at the token's
cache cell; head ``h`` attends with KV head ``h // (num_heads / num_kv_heads)``, scores times
``scale``, causal, optionally only the last ``window`` keys (src/iian/paged_attn.cpp:124), softmax in
float32; ``y = Wo concat(o)``.

The three projections run as one matrix product over the rows ``Wq | Wk | Wv`` stacked at load time.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import KVNeed, Mixer, POSITIONS, Prenormed, register_mixer


@register_mixer("attention")
class Attention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``, ``qk_norm``
    (bool), ``qk_norm_eps``, ``window`` (None or keys visible), ``position`` (a PartSpec)."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        if self.nkv <= 0 or self.nh % self.nkv:
            raise ValueError(f"attention: {self.nh} heads cannot share {self.nkv} KV heads")
        self.scale = float(p["scale"])
        self.qk_norm = bool(p.get("qk_norm", False))
        self.eps = float(p.get("qk_norm_eps", 0.0))
        self.window = p.get("window")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError("attention: window must be positive or None")
        self.position = POSITIONS.build(p["position"], dtype, device)
        if getattr(self.position, "dim", 0) > self.hd:
            raise ValueError(f"attention: position encoding rotates {self.position.dim} dims of a head of {self.hd}")
        self.q_size = self.nh * self.hd
        self.kv_size = self.nkv * self.hd
        self.w_qkv = self.w_o = self.b_qkv = self.b_o = self.q_norm_w = self.k_norm_w = None

    def tensors(self) -> Dict[str, TensorSpec]:
        t = {
            "q_proj.weight": TensorSpec((self.q_size, self.hidden)),
            "k_proj.weight": TensorSpec((self.kv_size, self.hidden)),
            "v_proj.weight": TensorSpec((self.kv_size, self.hidden)),
            "o_proj.weight": TensorSpec((self.hidden, self.q_size)),
            "q_proj.bias": TensorSpec((self.q_size,), optional=True, init="zeros"),
            "k_proj.bias": TensorSpec((self.kv_size,), optional=True, init="zeros"),
            "v_proj.bias": TensorSpec((self.kv_size,), optional=True, init="zeros"),
            "o_proj.bias": TensorSpec((self.hidden,), optional=True, init="zeros"),
        }
        if self.qk_norm:
            t["q_norm.weight"] = TensorSpec((self.hd,), init="ones_jitter")
            t["k_norm.weight"] = TensorSpec((self.hd,), init="ones_jitter")
        return t

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        ws = [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_qkv = torch.cat(ws, dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()
        if any(f"{n}_proj.bias" in tensors for n in "qkv"):
            parts = []
            for n, size in (("q", self.q_size), ("k", self.kv_size), ("v", self.kv_size)):
                b = tensors.get(f"{n}_proj.bias")
                parts.append(b.to(torch.float32) if b is not None else torch.zeros(size, dtype=torch.float32, device=self.device))
            self.b_qkv = torch.cat(parts).contiguous()
        if "o_proj.bias" in tensors:
            self.b_o = tensors["o_proj.bias"].to(torch.float32).contiguous()
        if self.qk_norm:
            self.q_norm_w = tensors["q_norm.weight"].to(torch.float32).contiguous()
            self.k_norm_w = tensors["k_norm.weight"].to(torch.float32).contiguous()

    def graph_plan(self, num_seqs: int, max_ctx: int):
        """The number of key splits of decode attention is part of a captured graph (grid and cluster sizes)."""
        k = ops.kernels()
        if not hasattr(k, "attention_splits"):
            return None
        return {"n_split": k.attention_splits(num_seqs, self.nkv, max_ctx)}

    def cache_need(self) -> KVNeed:
        return KVNeed(self.nkv, self.hd, int(self.window) if self.window is not None else None)

    def kernel_libraries(self):
        return ("rope_kv", "attention_generic", "gemm_simt")

    folds_norm_out = True

    def takes_prenormed(self, n_rows: int) -> bool:
        k = ops.kernels()
        return hasattr(k, "can_take_prenormed") and k.can_take_prenormed(n_rows, self.w_qkv, self.dtype)

    def _project_out(self, k, attn: torch.Tensor, ctx, norm_out):
        if (norm_out is not None and self.b_o is None and hasattr(k, "can_fuse_norm")
                and k.can_fuse_norm(attn, self.w_o)):
            return norm_out.take(k, attn, self.w_o, ctx)
        out = ctx.buf("mixer_out", (attn.shape[0], self.hidden), self.dtype)
        k.linear(attn, self.w_o, out)
        if self.b_o is not None:
            k.add_bias(out, self.b_o)
        return out

    def forward(self, x, ctx, cache, writes_cache: bool, norm_out=None):
        k = ops.kernels()
        scale = None
        if isinstance(x, Prenormed):
            x, scale = x.x, x.scale
        n = x.shape[0]
        pos = self.position
        if writes_cache:
            w, bias, nkv = self.w_qkv, self.b_qkv, self.nkv
        else:   # reads a cache another call filled: only Q is needed
            w, nkv = self.w_qkv[: self.q_size], 0
            bias = self.b_qkv[: self.q_size] if self.b_qkv is not None else None
        width = self.q_size + 2 * nkv * self.hd
        qkv = ctx.buf("qkv", (n, width), self.dtype)
        if scale is not None:
            k.linear(x, w, qkv, row_scale=scale)
        else:
            k.linear(x, w, qkv)
        if not pos.fused:
            pos.apply(qkv, self.nh, nkv, self.hd, ctx)
        meta = ctx.page_meta(cache.group)
        plan = ctx.graph_plan(self)
        n_split = plan["n_split"] if plan else None         # fixed inside a captured graph, else chosen per launch
        attn = ctx.buf("attn", (n, self.q_size), self.dtype)
        rot_dim = pos.dim if pos.fused else 0
        table = pos.table(ctx) if pos.fused and hasattr(pos, "table") and pos.inv_freq is not None else None
        if (writes_cache and hasattr(k, "can_fuse_decode_attention") and (rot_dim == 0 or table is not None)
                and k.can_fuse_decode_attention(qkv, meta, num_heads=self.nh, num_kv_heads=self.nkv, head_dim=self.hd,
                                                rot_dim=rot_dim, rope_style=pos.style if pos.fused else 0, bias=bias)):
            # a decode step: norm, rotation, cache write and attention in one kernel
            k.attention_decode_fused(qkv, cache.k, cache.v, attn, meta, num_heads=self.nh, num_kv_heads=self.nkv,
                                     head_dim=self.hd, scale=self.scale, window=self.window,
                                     q_weight=self.q_norm_w, k_weight=self.k_norm_w, eps=self.eps,
                                     table=table if rot_dim else None, slots=meta.slots, write_kv=True, n_split=n_split)
            return self._project_out(k, attn, ctx, norm_out)
        q = ctx.buf("q", (n, self.nh, self.hd), self.dtype)
        k.qk_norm_rope_store(
            qkv, q, cache.k if writes_cache else None, cache.v if writes_cache else None,
            num_heads=self.nh, num_kv_heads=nkv, head_dim=self.hd,
            q_weight=self.q_norm_w, k_weight=self.k_norm_w, eps=self.eps,
            inv_freq=pos.inv_freq if pos.fused else None, rot_dim=pos.dim if pos.fused else 0,
            rope_style=pos.style if pos.fused else 0,
            positions=ctx.positions, slots=meta.slots if writes_cache else None, write_kv=writes_cache, bias=bias,
            **({"table": table} if table is not None else {}))
        k.paged_attention(q, cache.k, cache.v, attn, meta, num_heads=self.nh, num_kv_heads=self.nkv,
                          head_dim=self.hd, scale=self.scale, window=self.window, n_split=n_split)
        return self._project_out(k, attn, ctx, norm_out)
