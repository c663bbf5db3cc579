"""Position encodings.

``rotary``: rotation of pairs of the head by angles ``pos * base^(-2j/dim)``
(third_party/ggml/src/ggml-cpu/ops.cpp:5958-5990; pairing styles :6063-6079).  The part owns the
float32 table of ``base^(-2j/dim)``; the attention mixer hands it to the fused kernel, which
multiplies by the position and takes sin/cos in float32.  ``dim`` may be smaller than the head
(partial rotation); Qwen3 rotates the whole head (src/iian/arch/qwen3.cpp:66).

``none``: no position signal (the mixer stores K unrotated).

Another encoding is another class registered with ``register_position``.  If it cannot be expressed
as a rotation table it sets ``fused = False`` and implements ``apply(q, k, positions, ctx)``, which the
attention mixer calls on the projected heads before they are stored.
"""
from __future__ import annotations

import torch

from .base import PositionEncoding, register_position

ROPE_STYLES = {"neox": 0, "interleaved": 1}


@register_position("rotary")
class Rotary(PositionEncoding):
    """params: ``dim`` (rotated dims, even), ``base``, ``style`` (``neox`` pairs (j, j+dim/2),
    ``interleaved`` pairs (2j, 2j+1)), ``max_position``; optional ``frequency_scale`` (linear scaling,
    the reference's ``freq_scale``, default 1)."""

    fused = True

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.dim = int(spec["dim"])
        if self.dim <= 0 or self.dim % 2:
            raise ValueError(f"rotary: dim must be positive and even, got {self.dim}")
        self.base = float(spec["base"])
        style = spec.params.get("style", "neox")
        if style not in ROPE_STYLES:
            raise ValueError(f"rotary: unknown style '{style}' ({', '.join(ROPE_STYLES)})")
        self.style = ROPE_STYLES[style]
        self.max_position = int(spec.params.get("max_position", 0))
        scale = float(spec.params.get("frequency_scale", 1.0))
        j = torch.arange(self.dim // 2, dtype=torch.float64)
        inv = scale * torch.pow(torch.tensor(self.base, dtype=torch.float64), -2.0 * j / self.dim)
        self.inv_freq = inv.to(torch.float32).to(device)
        self.key = ("rotary", self.dim, self.base, scale)

    def table(self, ctx):
        """cos and sin of this step's angles, float32 [N, dim / 2, 2].  The angles depend on the positions
        and on this part's constants only, so one table per step serves every layer that rotates alike."""
        from .. import ops
        tables = ctx.step_cache.setdefault("rotary_tables", {}) if hasattr(ctx, "step_cache") else {}
        t = tables.get(self.key)
        if t is None:
            k = ops.kernels()
            if not hasattr(k, "rotary_table"):
                return None
            n = ctx.positions.shape[0]
            t = ctx.buf(f"rotary_table_{len(tables)}", (n, self.dim // 2, 2), torch.float32)
            k.rotary_table(self.inv_freq, ctx.positions, self.dim // 2, t)
            tables[self.key] = t
        return t


@register_position("none")
class NoPosition(PositionEncoding):
    fused = True
    dim = 0
    style = 0
    inv_freq = None
