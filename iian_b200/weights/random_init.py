"""Random weights from a configuration and a seed.

The reference has no such mode (every test of it needs a real checkpoint, CLAUDE.md:13-17;
its bench randomises token ids only, src/iian/cli/cmd_bench.cpp:58-65).  Here a model folder
(``config.json`` + ``model.safetensors``) can be written from a configuration alone, and the
same generator can fill a model directly on the device for large shapes.

Matrices are N(0, std); norm weights are ``1 + U(-jitter, jitter)``; each tensor has a
generator of its own keyed by ``(seed, name)``, so a tensor's values do not depend on which
other tensors exist.  Values drawn on the CPU and on a GPU differ (different generators).
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict, Mapping, Optional

import torch

from .loader import TensorSpec, WeightSource, kept_dtype
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 0x9E3779B1 + zlib.crc32(name.encode("utf-8"))) & 0x7FFFFFFFFFFFFFFF


def draw(name: str, spec: TensorSpec, seed: int, device: torch.device, std: float, jitter: float) -> torch.Tensor:
    """One tensor in float32 on ``device``."""
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    if spec.kind == "int":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if spec.init == "ones_jitter":
        t = torch.rand(spec.shape, generator=gen, device=device, dtype=torch.float32)
        return 1.0 + (2.0 * t - 1.0) * jitter
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=torch.float32, device=device)
    t = torch.empty(spec.shape, device=device, dtype=torch.float32)
    # fill large tensors in slabs to bound the temporary memory
    flat = t.view(-1)
    step = 1 << 28
    for s in range(0, flat.numel(), step):
        flat[s:s + step].normal_(0.0, std, generator=gen)
    return t


class RandomWeights(WeightSource):
    """Declared tensors filled from a seed.  Optional tensors (biases) are left out unless
    ``with_optional`` is set."""

    def __init__(self, seed: int, std: float = 0.02, norm_jitter: float = 0.1,
                 store_dtype: torch.dtype = torch.bfloat16, with_optional: bool = False):
        self.seed = seed
        self.std = std
        self.norm_jitter = norm_jitter
        self.store_dtype = store_dtype
        self.with_optional = with_optional
        self._declared: Mapping[str, TensorSpec] = {}

    def describe(self) -> str:
        return f"random weights (seed {self.seed})"

    def check(self, declared: Mapping[str, TensorSpec]) -> None:
        self._declared = declared

    def has(self, name: str) -> bool:
        spec = self._declared.get(name)
        return spec is not None and (self.with_optional or not spec.optional)

    def stored_dtype(self, spec: TensorSpec) -> torch.dtype:
        """Matrices in ``store_dtype``; norm weights in float32 (a tensor stored in 32 bits)."""
        if spec.kind == "int":
            return torch.int32
        return torch.float32 if spec.init == "ones_jitter" else self.store_dtype

    def fetch(self, name: str, spec: TensorSpec, compute: torch.dtype, device: torch.device) -> torch.Tensor:
        t = draw(name, spec, self.seed, device, self.std, self.norm_jitter)
        stored = self.stored_dtype(spec)
        t = t.to(stored)                      # round once, as a file would hold it
        return t.to(kept_dtype(stored, spec.kind, compute)).contiguous()


def write_model_folder(out_dir: str, architecture, config, seed: int, *, std: float = 0.02,
                       norm_jitter: float = 0.1, store_dtype: torch.dtype = torch.bfloat16,
                       with_optional: bool = False) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with random weights."""
    from ..engine.model import declare_tensors     # parts are only needed for their declarations

    os.makedirs(out_dir, exist_ok=True)
    spec = architecture.build_spec(config)
    declared = declare_tensors(architecture, spec)
    src = RandomWeights(seed, std, norm_jitter, store_dtype, with_optional)
    src.check(declared)
    cpu = torch.device("cpu")
    tensors: Dict[str, torch.Tensor] = {}
    for name, tspec in declared.items():
        if not src.has(name):
            continue
        tensors[name] = draw(name, tspec, seed, cpu, std, norm_jitter).to(src.stored_dtype(tspec))
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(architecture.config_to_dict(config), f, indent=2)
    return out_dir
