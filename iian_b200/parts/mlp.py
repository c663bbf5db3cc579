"""Dense gated feed-forward: ``y = Wdown (act(Wgate h) * (Wup h))``, parallel gate, no biases
(src/iian/graph.cpp:116-163 with ``FfnOp::SILU`` / ``FfnGate::PAR``, src/iian/arch/qwen3.cpp:97).
``silu(z) = z / (1 + exp(-z))`` (third_party/ggml/src/ggml-cpu/vec.h:1046-1048).

Gate and up projections run as one matrix product over the rows of both, stacked at load time in groups of
8 (8 gate rows, then the 8 up rows of the same features, ...), so that a product kernel that owns 16
consecutive rows holds both halves of 8 features and can apply SiLU(gate) * up in its epilogue.  If the
intermediate size is no multiple of 8 the rows are stacked as ``Wgate | Wup``.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import FeedForward, Prenormed, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    """params: ``hidden_size``, ``intermediate_size``, ``activation`` (``silu``)."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        act = spec.params.get("activation", "silu")
        if act != "silu":
            raise ValueError(f"gated_mlp: activation '{act}' has no kernel (silu only)")
        self.w_gate_up = self.w_down = None
        self.interleave = 0

    def tensors(self) -> Dict[str, TensorSpec]:
        return {
            "gate_proj.weight": TensorSpec((self.inter, self.hidden)),
            "up_proj.weight": TensorSpec((self.inter, self.hidden)),
            "down_proj.weight": TensorSpec((self.hidden, self.inter)),
        }

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        if self.inter % 8 == 0:
            k = g.shape[1]
            self.w_gate_up = torch.stack([g.view(self.inter // 8, 8, k), u.view(self.inter // 8, 8, k)], dim=1) \
                .reshape(2 * self.inter, k).contiguous()
            self.interleave = 8
        else:
            self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
            self.interleave = 0
        self.w_down = tensors["down_proj.weight"].contiguous()

    def kernel_libraries(self):
        return ("elementwise", "gemm_simt")

    folds_norm_out = True

    def takes_prenormed(self, n_rows: int) -> bool:
        k = ops.kernels()
        return (hasattr(k, "can_take_prenormed") and self.interleave == 8
                and k.can_take_prenormed(n_rows, self.w_gate_up, self.dtype))

    def forward(self, x, ctx, norm_out=None):
        k = ops.kernels()
        scale = None
        if isinstance(x, Prenormed):
            x, scale = x.x, x.scale
        n = x.shape[0]
        act = ctx.buf("ffn_act", (n, self.inter), self.dtype)
        if scale is not None:
            k.linear_swiglu(x, self.w_gate_up, act, row_scale=scale)
        elif hasattr(k, "can_fuse_swiglu") and k.can_fuse_swiglu(x, self.w_gate_up, self.interleave):
            k.linear_swiglu(x, self.w_gate_up, act)            # the activation rides in the product's epilogue
        else:
            gate_up = ctx.buf("gate_up", (n, 2 * self.inter), self.dtype)
            k.linear(x, self.w_gate_up, gate_up)
            k.swiglu(gate_up, act, self.interleave)
        if norm_out is not None and hasattr(k, "can_fuse_norm") and k.can_fuse_norm(act, self.w_down):
            return norm_out.take(k, act, self.w_down, ctx)
        out = ctx.buf("ffn_out", (n, self.hidden), self.dtype)
        k.linear(act, self.w_down, out)
        return out
