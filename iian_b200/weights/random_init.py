"""Random weights from a configuration and a seed.

The reference has no such mode (every test of it needs a real checkpoint, CLAUDE.md:13-17;
its bench randomises token ids only, src/iian/cli/cmd_bench.cpp:58-65).  Here a model folder
(``config.json`` + ``model.safetensors``) can be written from a configuration alone, and the
same generator can fill a model directly on the device for large shapes.

Matrices are N(0, std); norm weights are ``1 + U(-jitter, jitter)``.  Every element is a function of
``(seed, tensor name, element index)`` alone -- a counter-based generator, written with integer and
IEEE-exact floating operations only -- so a tensor's values do not depend on which other tensors exist,
on the device they are drawn on (CPU and GPU give the same bits), or on how the work is cut into slabs.
A plain implementation on the CPU can therefore rebuild the model a GPU run used from the seed alone.

Element ``i`` of tensor ``name``: ``h = mix(key ^ i * odd)`` with ``key = mix(seed) ^ fnv1a(name)`` and
``mix`` the SplitMix64 finaliser.  A uniform takes the top 24 bits of ``h``.  A normal takes the top 32
bits ``u``: ``t = KNOTS[u >> 16]``, ``x = t + (KNOTS[(u >> 16) + 1] - t) * ((u & 0xFFFF) / 65536)`` with
``KNOTS[k] = probit((k + 0.5) / 65537)`` held in float32: the inverse normal distribution function by
linear interpolation in a table, so no transcendental function is evaluated per element (their last
bits differ between CPU and GPU libraries); the tails end near 4.3 standard deviations.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Mapping, Optional

import torch

from .loader import TensorSpec, WeightSource, kept_dtype
from .safetensors_io import write_safetensors

_M64 = (1 << 64) - 1


def _s64(x: int) -> int:
    """A 64-bit pattern as the signed integer torch's int64 holds."""
    x &= _M64
    return x - (1 << 64) if x >= (1 << 63) else x


def _mix_int(x: int) -> int:
    """SplitMix64's finaliser on a Python integer."""
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def _fnv1a(name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & _M64
    return h


def tensor_key(seed: int, name: str) -> int:
    return _mix_int(int(seed) & _M64) ^ _fnv1a(name)


def _lsr(x: torch.Tensor, k: int) -> torch.Tensor:
    """Logical shift right of int64 lanes (torch's ``>>`` keeps the sign)."""
    return (x >> k) & ((1 << (64 - k)) - 1)


def _mix(x: torch.Tensor) -> torch.Tensor:
    """SplitMix64's finaliser on int64 lanes; multiplication wraps modulo 2^64 on the CPU and on CUDA alike."""
    x = x + _s64(0x9E3779B97F4A7C15)
    x = (x ^ _lsr(x, 30)) * _s64(0xBF58476D1CE4E5B9)
    x = (x ^ _lsr(x, 27)) * _s64(0x94D049BB133111EB)
    return x ^ _lsr(x, 31)


def element_bits(key: int, start: int, count: int, device: torch.device) -> torch.Tensor:
    """The 64 random bits of elements ``start .. start + count`` of the tensor with ``key`` (int64 lanes)."""
    i = torch.arange(start, start + count, dtype=torch.int64, device=device)
    return _mix((i * _s64(0xD1B54A32D192ED03)) ^ _s64(key))


_KNOTS: Dict[torch.device, torch.Tensor] = {}


def _knots(device: torch.device) -> torch.Tensor:
    t = _KNOTS.get(device)
    if t is None:
        p = (torch.arange(65537, dtype=torch.float64) + 0.5) / 65537.0
        t = (torch.special.ndtri(p)).to(torch.float32).to(device)       # computed on the CPU whatever the device
        _KNOTS[device] = t
    return t


def uniform(key: int, start: int, count: int, device: torch.device) -> torch.Tensor:
    """float32 in [0, 1): the top 24 bits of each element's hash."""
    return _lsr(element_bits(key, start, count, device), 40).to(torch.float32) * (1.0 / (1 << 24))


def standard_normal(key: int, start: int, count: int, device: torch.device) -> torch.Tensor:
    u = _lsr(element_bits(key, start, count, device), 32)
    knots = _knots(device)
    cell = u >> 16
    lo = knots[cell]
    hi = knots[cell + 1]
    frac = (u & 0xFFFF).to(torch.float32) * (1.0 / 65536.0)
    return lo + (hi - lo) * frac                    # separate multiply and add: no fused rounding on either device


def draw(name: str, spec: TensorSpec, seed: int, device: torch.device, std: float, jitter: float) -> torch.Tensor:
    """One tensor in float32 on ``device``."""
    if spec.kind == "int":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=torch.float32, device=device)
    key = tensor_key(seed, name)
    t = torch.empty(spec.shape, device=device, dtype=torch.float32)
    flat = t.view(-1)
    step = 1 << 24                                  # slabs bound the temporary memory (a few hundred MB)
    for s in range(0, flat.numel(), step):
        n = min(step, flat.numel() - s)
        if spec.init == "ones_jitter":
            flat[s:s + n] = 1.0 + (2.0 * uniform(key, s, n, device) - 1.0) * jitter
        else:
            flat[s:s + n] = standard_normal(key, s, n, device) * std
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
                       with_optional: bool = False, device: str = "cpu") -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with random weights.  ``device`` is where
    the values are drawn (the file is the same whichever it is; a GPU is faster for large shapes)."""
    from ..engine.model import declare_tensors     # parts are only needed for their declarations

    os.makedirs(out_dir, exist_ok=True)
    spec = architecture.build_spec(config)
    declared = declare_tensors(architecture, spec)
    src = RandomWeights(seed, std, norm_jitter, store_dtype, with_optional)
    src.check(declared)
    dev = torch.device(device)
    tensors: Dict[str, torch.Tensor] = {}
    for name, tspec in declared.items():
        if not src.has(name):
            continue
        tensors[name] = draw(name, tspec, seed, dev, std, norm_jitter).to(src.stored_dtype(tspec)).cpu()
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(architecture.config_to_dict(config), f, indent=2)
    return out_dir
