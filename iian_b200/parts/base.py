"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from a :class:`~iian_b200.config.spec.PartSpec` (its sizes and constants), the
activation dtype and the device.  It declares the tensors it needs under names local to itself
(:meth:`Part.tensors`), receives them (:meth:`Part.bind`), and computes through
``iian_b200.ops.kernels()``.  It never sees the model's configuration.

The reference has the same inventory as methods of one ``GraphContext`` (include/iian/graph.h:60-150:
``build_norm``, ``build_qkv``, ``build_rope``, ``build_attn``, ``build_ffn``, ``build_lm_head``) that
read several constants from a shared hyper-parameter struct (src/iian/graph.cpp:25-30, :107); here
each kind is a class chosen by name, layer by layer.

Interfaces
----------
``Norm.forward(residual, delta, ctx) -> normed``
    ``residual`` is the float32 residual stream ``[N, H]``; if ``delta`` is given it is first added
    into ``residual`` in place (the residual sum is always float32).  Returns the normalised rows in
    the activation dtype.
``Mixer.forward(x, ctx, cache, writes_cache) -> y``
    ``x``: normalised rows ``[N, H]``; ``cache``: what :meth:`Mixer.cache_need` asked for (a
    :class:`~iian_b200.cache.storage.KVView`, a :class:`~iian_b200.cache.storage.StateView` or
    None); ``writes_cache`` is False when the run order lets this call read another call's cache.
    Returns ``[N, H]`` in the activation dtype.
``FeedForward.forward(x, ctx) -> y``
    rows in, rows out, ``[N, H]``.
``PositionEncoding``
    owned by the mixer that needs positions; the attention mixer asks it for the rotation table.
``Embedding.forward(tokens, ctx) -> residual`` and ``Head.forward(x, ctx) -> logits`` (float32).

Optional: a norm folded into its neighbours
-------------------------------------------
A norm that is a factor per row and a weight per column (RMSNorm) can be carried by the matrix products on
either side of it (``iian_b200.ops.fused``).  The arrangement offers this to parts that declare support:

* a norm with ``foldable() -> (weight, eps)`` may be folded;
* a mixer or feed-forward with ``folds_norm_out = True`` accepts ``forward(..., norm_out=request)`` where
  ``request`` is a :class:`NormOut`; if its last product can carry it, it calls ``request.take(...)`` and returns
  a :class:`Prenormed` instead of rows; otherwise it ignores the request and returns rows as usual;
* a mixer or feed-forward with ``takes_prenormed(n_rows) -> bool`` true may be handed a :class:`Prenormed` as
  ``x``: rows that still lack the factor per row, with the sums of squares from which its first product takes it.

A part that declares none of this (the default) is always called with plain rows.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple, Type

import torch

from ..config.spec import PartSpec
from ..weights.loader import TensorSpec


@dataclass(frozen=True)
class KVNeed:
    """Per-token entries: keys and values of ``num_kv_heads`` heads of ``head_dim``; ``window`` = how
    many of the latest keys stay needed (None: all)."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size state per request: one tensor of ``shape`` and ``dtype`` per slot.

    The state after token t depends on every token before it and only its latest value is kept, so a
    request cannot start behind a prefix that another request computed: a model with such a need runs
    with prefix reuse switched off (``prefix_reusable``)."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


def prefix_reusable(need) -> bool:
    """Whether a request may skip tokens whose cache entries another request left behind.  Keys and values
    per token can be shared page by page; a fixed-size state cannot (it would need a snapshot per page)."""
    return isinstance(need, KVNeed)


class Part:
    def __init__(self, spec: PartSpec, dtype: torch.dtype, device: torch.device):
        self.spec = spec
        self.dtype = dtype
        self.device = device

    def tensors(self) -> Dict[str, TensorSpec]:
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass

    def kernel_libraries(self) -> Tuple[str, ...]:
        """Names of the CUDA libraries this part launches (compiled together before the first step)."""
        return ()

    # Whether ``forward`` may be recorded into a CUDA graph and replayed for later steps: it must read the
    # step's integers from the context's device tensors only (never from the host lists ``h_*``, whose values
    # a recording would freeze), launch the same work whatever those integers are, and leave padding rows
    # (sequence -1, cache cell -1, state slot -1) without effect.  A model with a part that says False runs
    # its decode steps eagerly.
    graph_safe = True


@dataclass
class Prenormed:
    """The input of a sub-layer whose norm rides in the surrounding products: ``x`` = residual * norm weight in
    the activation dtype, ``scale`` the ``ops.fused.RowScale`` that completes it, ``norm`` the norm part it
    stands for (the residual stream already holds the sum that norm would have added)."""
    x: torch.Tensor
    scale: object
    norm: object


@dataclass
class NormOut:
    """A request to the part that ends a sub-layer: add your output to ``residual`` and prepare the input of
    ``norm`` (weight ``weight``, ``eps``) in your last product."""
    residual: torch.Tensor
    norm: object
    weight: torch.Tensor
    eps: float
    name: str                   # distinguishes the buffers of the two sub-layers of a block

    def take(self, k, x: torch.Tensor, w: torch.Tensor, ctx) -> "Prenormed":
        """Run ``x @ w.T`` with the folded epilogue and return what the next sub-layer gets."""
        from ..ops.fused import ResidualNorm, RowScale
        n, width = x.shape[0], w.shape[0]
        out = ctx.buf(f"prenormed_{self.name}", (n, width), x.dtype)
        partials = ctx.buf(f"norm_partials_{self.name}", (n, k.norm_parts(w, n)), torch.float32)
        k.linear(x, w, out, residual_norm=ResidualNorm(self.residual, self.weight, partials))
        return Prenormed(out, RowScale(partials, width, self.eps), self.norm)


class Norm(Part):
    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], ctx) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError

    def foldable(self):
        """(weight float32 [H], eps) if this norm is ``x * rsqrt(mean(x^2) + eps) * weight``, else None."""
        return None


class Mixer(Part):
    folds_norm_out = False

    def takes_prenormed(self, n_rows: int) -> bool:
        return False

    def cache_need(self):
        return None

    def graph_plan(self, num_seqs: int, max_ctx: int):
        """What this mixer must keep fixed inside a captured graph for ``num_seqs`` sequences of one token with
        contexts up to ``max_ctx`` (grid sizes, split counts: anything it would otherwise derive from the step's host
        values), or None.  The runner asks once per captured graph and hands the answer back through
        ``ctx.graph_plan(self)`` on every replayed step; on eager steps that returns None."""
        return None

    def forward(self, x: torch.Tensor, ctx, cache, writes_cache: bool) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError


class FeedForward(Part):
    folds_norm_out = False

    def takes_prenormed(self, n_rows: int) -> bool:
        return False

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError


class PositionEncoding(Part):
    pass


class Embedding(Part):
    def forward(self, tokens: torch.Tensor, ctx) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError


class Head(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._kinds: Dict[str, Type[Part]] = {}

    def register(self, kind: str) -> Callable[[Type[Part]], Type[Part]]:
        def deco(cls: Type[Part]) -> Type[Part]:
            self._kinds[kind] = cls
            return cls
        return deco

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def build(self, spec: PartSpec, dtype: torch.dtype, device: torch.device) -> Part:
        try:
            cls = self._kinds[spec.kind]
        except KeyError:
            raise KeyError(f"unknown {self.what} '{spec.kind}'; registered: {', '.join(sorted(self._kinds))}") from None
        return cls(spec, dtype, device)

    def kinds(self):
        return sorted(self._kinds)


NORMS = Registry("norm")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
POSITIONS = Registry("position encoding")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")
BLOCKS: Dict[str, type] = {}

register_norm = NORMS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_position = POSITIONS.register
register_embedding = EMBEDDINGS.register
register_head = HEADS.register


def register_block(kind: str):
    def deco(cls):
        BLOCKS[kind] = cls
        return cls
    return deco
