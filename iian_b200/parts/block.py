"""How a layer's parts are arranged.

A block implements one arrangement (``LayerSpec.arrangement``) and is registered under its name with
``register_block``.  What the model asks of a block: ``__init__(spec, dtype, device)`` builds its parts from the
slots of the ``LayerSpec`` it understands; ``parts()`` lists them with the slot names their tensors go under;
``cache_need()`` says what the cache of a call to this layer must hold (a ``KVNeed``, a ``StateNeed`` or None);
``forward(residual, delta, ctx, cache, writes_cache, select_rows)`` takes the float32 residual stream and the
not-yet-added output of whatever ran before, and returns the same pair.

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
from .base import FEED_FORWARDS, MIXERS, NORMS, NormOut, Prenormed, register_block


@register_block("pre_norm_residual")
class PreNormResidualBlock:
    def __init__(self, spec: LayerSpec, dtype: torch.dtype, device: torch.device):
        missing = [s for s in ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm") if spec.slot(s) is None]
        if missing:
            raise ValueError(f"arrangement pre_norm_residual needs the slots {', '.join(missing)}")
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

    def cache_need(self):
        return self.mixer.cache_need()

    accepts_next_norm = True

    @staticmethod
    def _norm_out(norm, consumer, residual: torch.Tensor, n_rows: int, name: str) -> Optional[NormOut]:
        """A request to fold ``norm`` into the products around it, if the norm allows it and ``consumer`` (the part
        that follows it) can take rows that still lack the factor per row."""
        if norm is None or consumer is None:
            return None
        fold = norm.foldable()
        if fold is None or not consumer.takes_prenormed(n_rows):
            return None
        return NormOut(residual, norm, fold[0], fold[1], name)

    def forward(self, residual: torch.Tensor, delta, ctx, cache, writes_cache: bool,
                select_rows: Optional[torch.Tensor], next_norm=None, next_consumer=None):
        """``delta`` is the not-yet-added output of the sub-layer before this block, or a ``Prenormed`` for this
        block's first norm (then the sum is already in ``residual``).  ``next_norm`` / ``next_consumer``: the norm
        and the part that follow this block's feed-forward, if its last product may prepare their input."""
        if isinstance(delta, Prenormed):
            if delta.norm is not self.mixer_norm:
                raise RuntimeError("block: received rows prepared for another norm")
            h = delta
        else:
            h = self.mixer_norm.forward(residual, delta, ctx)
        n_rows = residual.shape[0]
        gathers = select_rows is not None and not getattr(ctx, "rows_identity", False)
        request = None
        if not gathers and self.mixer.folds_norm_out:
            request = self._norm_out(self.feed_forward_norm, self.feed_forward, residual, n_rows, "mixer")
        y = self.mixer.forward(h, ctx, cache, writes_cache, norm_out=request) if request is not None \
            else self.mixer.forward(h, ctx, cache, writes_cache)
        if gathers:
            k = ops.kernels()
            r = select_rows.shape[0]
            res_sel = ctx.buf("residual_rows", (r, residual.shape[1]), residual.dtype)
            y_sel = ctx.buf("mixer_out_rows", (r, y.shape[1]), y.dtype)
            k.gather_rows(residual, select_rows, res_sel)
            k.gather_rows(y, select_rows, y_sel)
            residual, y = res_sel, y_sel
        h2 = y if isinstance(y, Prenormed) else self.feed_forward_norm.forward(residual, y, ctx)
        request = None
        if self.feed_forward.folds_norm_out:
            request = self._norm_out(next_norm, next_consumer, residual, residual.shape[0], "feed_forward")
        d = self.feed_forward.forward(h2, ctx, norm_out=request) if request is not None else self.feed_forward.forward(h2, ctx)
        return residual, d
