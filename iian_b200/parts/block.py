"""How a layer's parts are arranged.

``pre_norm_residual`` (src/iian/arch/qwen3.cpp:74-100): ``x += mixer(norm(x))``; ``x += ffn(norm(x))``.
The add that closes one sub-layer is fused into the norm that opens the next: a block receives the
float32 residual and the not-yet-added output of the previous sub-layer (``delta``) and returns the
same pair.

Row selection: in the last entry of the run order only the rows whose logits are wanted go on after
the mixer -- both the mixer's output and the residual (src/iian/arch/qwen3.cpp:91,
src/iian/graph.cpp:356-358) -- so the last feed-forward, the final norm and the head run on those rows.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import ops
from ..config.spec import LayerSpec
from .base import FEED_FORWARDS, MIXERS, NORMS, register_block


@register_block("pre_norm_residual")
class PreNormResidualBlock:
    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device: torch.device):
        self.spec = spec
        self.dtype = dtype
        self.mixer_norm = NORMS.build(spec.mixer_norm, dtype, device)
        self.mixer = MIXERS.build(spec.mixer, dtype, device)
        self.feed_forward_norm = NORMS.build(spec.feed_forward_norm, dtype, device)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward, dtype, device)

    def parts(self):
        """(slot name, part) pairs; the slot name is what the architecture maps to file names."""
        return (("mixer_norm", self.mixer_norm), ("mixer", self.mixer),
                ("feed_forward_norm", self.feed_forward_norm), ("feed_forward", self.feed_forward))

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], ctx, cache, writes_cache: bool,
                select_rows: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        h = self.mixer_norm.forward(residual, delta, ctx)
        y = self.mixer.forward(h, ctx, cache, writes_cache)
        if select_rows is not None and not getattr(ctx, "rows_identity", False):
            k = ops.kernels()
            r = select_rows.shape[0]
            res_sel = ctx.buf("residual_rows", (r, residual.shape[1]), residual.dtype)
            y_sel = ctx.buf("mixer_out_rows", (r, y.shape[1]), y.dtype)
            k.gather_rows(residual, select_rows, res_sel)
            k.gather_rows(y, select_rows, y_sel)
            residual, y = res_sel, y_sel
        h2 = self.feed_forward_norm.forward(residual, y, ctx)
        d = self.feed_forward.forward(h2, ctx)
        return residual, d
