"""Descriptions of what a matrix product may do beyond the product itself.

RMSNorm is ``x * rsqrt(mean(x^2) + eps) * w`` (src/iian/graph.cpp:105-114): the weight acts per column, the
rest is one factor per row, and a factor per row commutes with a matrix product.  So the product that ends a
sub-layer can add its result to the residual stream, store ``residual * w`` for the next product and leave
the rows' sums of squares (:class:`ResidualNorm`), and the next product multiplies its rows by the factor
(:class:`RowScale`).  The norm kernel between them disappears; nothing is summed in a different precision
(residual and sums of squares stay float32).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class RowScale:
    """Row n of the product is multiplied by ``rsqrt(sum(partials[n]) / width + eps)``."""
    partials: torch.Tensor      # float32 [rows, parts]
    width: int
    eps: float


@dataclass
class ResidualNorm:
    """``residual += product`` (rounded to the activation dtype first); out = ``residual * weight``; the sums
    of squares of ``residual``'s rows go to ``partials`` in parts."""
    residual: torch.Tensor      # float32 [rows, width], updated in place
    weight: torch.Tensor        # float32 [width]
    partials: torch.Tensor      # float32 [rows, parts], written
