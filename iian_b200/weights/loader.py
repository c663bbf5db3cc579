"""Weights by tensor name: declaration, validation, placement.

Parts declare the tensors they need (:class:`TensorSpec`); the architecture gives each its
name in the file.  Loading checks the whole file against the declarations first and raises
ONE error that lists every missing tensor, every unexpected tensor and every wrong shape --
the reference raises on the first of each (src/iian/model_loader.cpp:181-184 missing,
:209-221 wrong shape, :207 declared twice) and only warns about unused tensors (:467-469).

Kept precision: a floating tensor stored in 16 bits is held as bfloat16; a tensor stored in
32 bits stays 32-bit; integer tables become int32.  With ``dtype=float32`` every floating
tensor is widened to 32 bits (exact), which is the engine's true 32-bit path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Mapping, Optional, Tuple

import torch

from .safetensors_io import TensorStore


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part needs.  ``kind``: ``"float"`` or ``"int"`` (integer table)."""

    shape: Tuple[int, ...]
    optional: bool = False
    kind: str = "float"
    init: str = "normal"          # how the random-weights mode fills it: normal | ones_jitter | zeros


class WeightsError(ValueError):
    """One message for everything wrong with a weight file."""

    def __init__(self, source: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_dtype: List[Tuple[str, str]] = ()):  # type: ignore[assignment]
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = [f"{source}: weights do not match the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: expected {list(e)}, got {list(g)}" for n, e, g in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtypes ({len(self.wrong_dtype)}): " + "; ".join(
                f"{n}: {why}" for n, why in self.wrong_dtype))
        super().__init__("\n".join(lines))


_FLOAT_TAGS = ("F64", "F32", "F16", "BF16")
_INT_TAGS = ("I64", "I32", "I16", "I8", "U8")


def kept_dtype(stored: torch.dtype, kind: str, compute: torch.dtype) -> torch.dtype:
    """The dtype a stored tensor is held in (see the module docstring)."""
    if kind == "int":
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


class WeightSource:
    """Where declared tensors come from."""

    def describe(self) -> str:  # pragma: no cover - interface
        raise NotImplementedError

    def check(self, declared: Mapping[str, TensorSpec]) -> None:  # pragma: no cover - interface
        raise NotImplementedError

    def has(self, name: str) -> bool:  # pragma: no cover - interface
        raise NotImplementedError

    def fetch(self, name: str, spec: TensorSpec, compute: torch.dtype, device: torch.device) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError


class FileWeights(WeightSource):
    """Tensors of a model folder's safetensors file(s)."""

    def __init__(self, model_dir: str):
        self.store = TensorStore(model_dir)
        self.model_dir = model_dir

    def describe(self) -> str:
        return self.model_dir

    def has(self, name: str) -> bool:
        return name in self.store.where

    def check(self, declared: Mapping[str, TensorSpec]) -> None:
        missing, unexpected, wrong_shape, wrong_dtype = [], [], [], []
        for name, spec in declared.items():
            if name not in self.store.where:
                if not spec.optional:
                    missing.append(name)
                continue
            ent = self.store.entry(name)
            if tuple(ent.shape) != tuple(spec.shape):
                wrong_shape.append((name, tuple(spec.shape), tuple(ent.shape)))
            if spec.kind == "float" and ent.dtype not in _FLOAT_TAGS:
                wrong_dtype.append((name, f"expected a floating type, file has {ent.dtype}"))
            if spec.kind == "int" and ent.dtype not in _INT_TAGS:
                wrong_dtype.append((name, f"expected an integer type, file has {ent.dtype}"))
        for name in self.store.names():
            if name not in declared:
                unexpected.append(name)
        if missing or unexpected or wrong_shape or wrong_dtype:
            raise WeightsError(self.model_dir, sorted(missing), sorted(unexpected), wrong_shape, wrong_dtype)

    def fetch(self, name: str, spec: TensorSpec, compute: torch.dtype, device: torch.device) -> torch.Tensor:
        t = self.store.read(name)
        return t.to(device=device, dtype=kept_dtype(t.dtype, spec.kind, compute)).contiguous()

    def close(self) -> None:
        self.store.close()


def load_declared(declared: Mapping[str, TensorSpec], source: WeightSource, compute: torch.dtype,
                  device: torch.device) -> Dict[str, torch.Tensor]:
    """Validate ``source`` against ``declared`` and return the tensors that exist."""
    source.check(declared)
    out: Dict[str, torch.Tensor] = {}
    for name, spec in declared.items():
        if source.has(name):
            out[name] = source.fetch(name, spec, compute, device)
    return out
