"""Architecture-neutral description of a model: which parts each layer is made of, and in
which order the layers run.

An architecture turns its typed configuration into a :class:`ModelSpec`.  Everything below
the architecture (parts, cache manager, step function) reads only the spec, so no part knows
which model it is in.  The reference keeps the same split between an architecture plug-in and
shared graph parts (include/iian/arch.h:22-34, include/iian/graph.h:60-150), but hands the
parts a global hyper-parameter struct; here every constant travels in ``PartSpec.params``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: ``kind`` selects the implementation in the part registry, ``params`` are
    its sizes and constants (never read from anywhere else)."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]


@dataclass(frozen=True)
class LayerSpec:
    """The parts of one layer and how they are arranged.

    ``arrangement`` names a block implementation (``"pre_norm_residual"``: x += mixer(norm(x));
    x += ffn(norm(x)), the order of src/iian/arch/qwen3.cpp:74-100).  The four named slots are what that
    arrangement uses; another arrangement takes the slots it needs (a slot it does not use stays ``None``) and may
    define further ones in ``extra`` as (slot name, part specification) pairs -- a norm after the mixer, a second
    mixer.  The block that implements the arrangement builds its parts from these and says under which slot names
    their tensors go (``parts()``).
    """

    mixer: Optional[PartSpec] = None
    feed_forward: Optional[PartSpec] = None
    mixer_norm: Optional[PartSpec] = None
    feed_forward_norm: Optional[PartSpec] = None
    arrangement: str = "pre_norm_residual"
    extra: Tuple[Tuple[str, PartSpec], ...] = ()

    def slot(self, name: str) -> Optional[PartSpec]:
        """The specification in slot ``name`` (one of the four named slots or one of ``extra``), or None."""
        if name in ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm"):
            return getattr(self, name)
        for n, spec in self.extra:
            if n == name:
                return spec
        return None


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be called more than once);
    ``cache`` is the cache this call's mixer works on.  A call that does not own its cache
    (``writes_cache=False``) reads what an earlier call with the same ``cache`` id stored.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding: PartSpec
    layers: Sequence[LayerSpec]
    order: Sequence[LayerCall]
    final_norm: PartSpec
    head: PartSpec

    def validate(self) -> None:
        owners: dict[int, int] = {}
        for idx, call in enumerate(self.order):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"run order entry {idx} names layer {call.layer}, "
                                 f"but the model has {len(self.layers)} layers")
            if call.writes_cache:
                if call.cache in owners:
                    raise ValueError(f"cache {call.cache} is written by run order entries "
                                     f"{owners[call.cache]} and {idx}")
                owners[call.cache] = idx
        for idx, call in enumerate(self.order):
            if not call.writes_cache:
                if call.cache not in owners:
                    raise ValueError(f"run order entry {idx} reads cache {call.cache}, which no entry writes")
                if owners[call.cache] > idx:
                    raise ValueError(f"run order entry {idx} reads cache {call.cache} before entry "
                                     f"{owners[call.cache]} has written it")
