"""A model: parts built from a :class:`ModelSpec`, weights bound by name, and the forward pass over
one step's tokens.

The reference splits this between ``ModelLoader::load`` (src/iian/model_loader.cpp:301-531: metadata
-> architecture -> declare and validate tensors by name -> upload) and the architecture's
``build_graph`` (src/iian/arch/qwen3.cpp:61-104).  Here the architecture only produces the spec and
the file names; the forward pass is the same loop for every architecture: embedding, the run order's
layer calls, final norm, head.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import parts as _parts  # noqa: F401  (registers the built-in parts)
from ..config.registry import Architecture, load_model_config
from ..config.spec import ModelSpec
from ..parts.base import BLOCKS, EMBEDDINGS, HEADS, NORMS
from ..weights.loader import FileWeights, TensorSpec, WeightSource, load_declared

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def resolve_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    try:
        return DTYPES[str(dtype)]
    except KeyError:
        raise ValueError(f"dtype must be 'bfloat16' or 'float32', got '{dtype}'") from None


def _scoped_parts(model_parts) -> List[Tuple[tuple, object]]:
    """Every part with the scope the architecture names its tensors by."""
    out = [(("embedding",), model_parts["embedding"])]
    for i, blk in enumerate(model_parts["blocks"]):
        for slot, part in blk.parts():
            out.append((("layer", i, slot), part))
    out.append((("final_norm",), model_parts["final_norm"]))
    out.append((("head",), model_parts["head"]))
    return out


def _build_parts(spec: ModelSpec, dtype: torch.dtype, device: torch.device):
    blocks = []
    for ls in spec.layers:
        try:
            cls = BLOCKS[ls.arrangement]
        except KeyError:
            raise KeyError(f"unknown block arrangement '{ls.arrangement}'; registered: {', '.join(sorted(BLOCKS))}") from None
        blocks.append(cls(ls, dtype, device))
    return {
        "embedding": EMBEDDINGS.build(spec.embedding, dtype, device),
        "blocks": blocks,
        "final_norm": NORMS.build(spec.final_norm, dtype, device),
        "head": HEADS.build(spec.head, dtype, device),
    }


def declare_tensors(arch: Architecture, spec: ModelSpec) -> Dict[str, TensorSpec]:
    """File name -> declaration for every tensor of the model (no device memory is touched)."""
    spec.validate()
    mp = _build_parts(spec, torch.float32, torch.device("meta"))
    declared: Dict[str, TensorSpec] = {}
    for scope, part in _scoped_parts(mp):
        for local, ts in part.tensors().items():
            name = arch.tensor_name(scope, local)
            if name in declared:
                raise ValueError(f"tensor '{name}' is declared twice")    # src/iian/model_loader.cpp:207
            declared[name] = ts
    return declared


class Model:
    def __init__(self, arch: Architecture, config, dtype, device, source: WeightSource):
        self.arch = arch
        self.config = config
        self.dtype = resolve_dtype(dtype)
        self.device = torch.device(device)
        self.spec = arch.build_spec(config)
        self.spec.validate()
        mp = _build_parts(self.spec, self.dtype, self.device)
        self.embedding = mp["embedding"]
        self.blocks = mp["blocks"]
        self.final_norm = mp["final_norm"]
        self.head = mp["head"]
        scoped = _scoped_parts(mp)
        declared: Dict[str, TensorSpec] = {}
        owner: Dict[str, Tuple[object, str]] = {}
        for scope, part in scoped:
            for local, ts in part.tensors().items():
                name = arch.tensor_name(scope, local)
                if name in declared:
                    raise ValueError(f"tensor '{name}' is declared twice")
                declared[name] = ts
                owner[name] = (part, local)
        loaded = load_declared(declared, source, self.dtype, self.device)
        per_part: Dict[int, Dict[str, torch.Tensor]] = {}
        for name, t in loaded.items():
            part, local = owner[name]
            per_part.setdefault(id(part), {})[local] = t
        self.weight_bytes = sum(t.numel() * t.element_size() for t in loaded.values())
        for _, part in scoped:
            part.bind(per_part.get(id(part), {}))
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding.weight)
        self.vocab_size = self.spec.vocab_size
        self.hidden_size = self.spec.hidden_size
        self.max_position = self.spec.max_position

    # ---- construction ----------------------------------------------------------------------
    @classmethod
    def from_folder(cls, model_dir: str, dtype="bfloat16", device="cuda:0") -> "Model":
        arch, config = load_model_config(model_dir)
        src = FileWeights(model_dir)
        try:
            return cls(arch, config, dtype, device, src)
        finally:
            src.close()

    @classmethod
    def from_random(cls, arch: Architecture, config, seed: int, dtype="bfloat16", device="cuda:0", **kw) -> "Model":
        from ..weights.random_init import RandomWeights
        return cls(arch, config, dtype, device, RandomWeights(seed, **kw))

    # ---- what the caches must provide -----------------------------------------------------
    def cache_needs(self) -> Dict[int, object]:
        """cache id -> KVNeed | StateNeed, taken from the mixer of the call that writes it."""
        needs: Dict[int, object] = {}

        def need_of(block):
            return block.cache_need() if hasattr(block, "cache_need") else block.mixer.cache_need()

        for call in self.spec.order:
            need = need_of(self.blocks[call.layer])
            if need is None:
                continue
            if call.writes_cache:
                needs[call.cache] = need
        for call in self.spec.order:
            if not call.writes_cache:
                need = need_of(self.blocks[call.layer])
                if need is not None and needs.get(call.cache) != need:
                    raise ValueError(f"layer {call.layer} reads cache {call.cache}, whose owner stores something else")
        return needs

    def all_parts(self) -> List[object]:
        out = [self.embedding, self.final_norm, self.head]
        for blk in self.blocks:
            out.extend(part for _, part in blk.parts())
        return out

    def graph_safe(self) -> bool:
        """Whether every part allows its forward pass to be replayed from a CUDA graph."""
        return all(getattr(part, "graph_safe", True) for part in self.all_parts())

    def kernel_libraries(self) -> List[str]:
        libs = set()
        for part in self.all_parts():
            libs.update(part.kernel_libraries())
        if self.dtype == torch.bfloat16:
            from ..csrc import build
            libs.update(build.BF16_SOURCES)
        return sorted(libs)

    # ---- one step ----------------------------------------------------------------------------
    def forward(self, ctx, storage) -> Optional[torch.Tensor]:
        """Run ``ctx.tokens`` through the model and return float32 logits ``[R, vocab]`` for
        ``ctx.out_rows`` (None if no row is wanted; the caches are still updated)."""
        if hasattr(ctx, "step_cache"):
            ctx.step_cache.clear()          # a context may be run twice (eagerly, then under graph capture)
        if self.device.type == "cuda":
            from ..ops.cuda_backend import pin_stream
            with pin_stream():
                return self._forward(ctx, storage)
        return self._forward(ctx, storage)

    def _forward(self, ctx, storage) -> Optional[torch.Tensor]:
        residual = self.embedding.forward(ctx.tokens, ctx)
        delta = None
        order = self.spec.order
        for idx, call in enumerate(order):
            select = ctx.out_rows if idx == len(order) - 1 else None
            block = self.blocks[call.layer]
            extra = {}
            if idx + 1 < len(order) and getattr(block, "accepts_next_norm", False):
                # the block after this one: its first norm may ride in this block's last product
                nxt = self.blocks[order[idx + 1].layer]
                if getattr(nxt, "accepts_next_norm", False):
                    extra = {"next_norm": nxt.mixer_norm, "next_consumer": nxt.mixer}
            residual, delta = block.forward(residual, delta, ctx, storage.view(call.cache), call.writes_cache, select, **extra)
        if not order:
            from .. import ops
            sel = ctx.buf("residual_rows", (ctx.out_rows.shape[0], residual.shape[1]), residual.dtype)
            ops.kernels().gather_rows(residual, ctx.out_rows, sel)
            residual = sel
        if ctx.out_rows.shape[0] == 0:
            return None
        normed = self.final_norm.forward(residual, delta, ctx)
        return self.head.forward(normed, ctx)
