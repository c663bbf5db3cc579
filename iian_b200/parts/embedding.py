"""Token embedding and output head.

Embedding: ``x0[t] = E[token_t]`` (src/iian/graph.cpp:39-46); the residual stream it starts is
float32.  Head: ``logits = Wout x`` in float32 on the rows asked for (src/iian/graph.cpp:360-376);
with tied embeddings ``Wout`` is the embedding table itself (src/iian/arch/qwen3.cpp:26-27).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Embedding, Head, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    """params: ``vocab_size``, ``hidden_size``."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.vocab = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab, self.hidden))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def kernel_libraries(self):
        return ("elementwise",)

    def forward(self, tokens: torch.Tensor, ctx) -> torch.Tensor:
        out = ctx.buf("residual", (tokens.shape[0], self.hidden), torch.float32)
        ops.kernels().embedding(self.weight, tokens, out)
        return out


@register_head("lm_head")
class LMHead(Head):
    """params: ``hidden_size``, ``vocab_size``, ``tied`` (use the embedding table)."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.vocab = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])
        self.tied = bool(spec.params.get("tied", False))
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorSpec]:
        return {} if self.tied else {"weight": TensorSpec((self.vocab, self.hidden))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = tensors["weight"].contiguous()

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table

    def kernel_libraries(self):
        return ("gemm_simt",)

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        logits = ctx.buf("logits", (x.shape[0], self.vocab), torch.float32)
        ops.kernels().linear(x, self.weight, logits)
        return logits
