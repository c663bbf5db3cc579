"""Reading and writing the safetensors container.

Layout: 8 bytes little-endian header length, a JSON header mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the
header), then the raw little-endian data.  The reference reads GGUF through a typed wrapper
with mmap (src/iian/gguf.cpp:16-84) and looks tensors up by name (gguf.cpp:222-225); this is
the same role for the file format this engine loads.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Optional, Tuple

import numpy as np
import torch

# safetensors dtype tag -> (torch dtype, numpy dtype used to view the bytes, bytes per element)
_DTYPES = {
    "F64": (torch.float64, np.dtype("<f8"), 8),
    "F32": (torch.float32, np.dtype("<f4"), 4),
    "F16": (torch.float16, np.dtype("<f2"), 2),
    "BF16": (torch.bfloat16, np.dtype("<u2"), 2),   # viewed as u16, reinterpreted by torch
    "I64": (torch.int64, np.dtype("<i8"), 8),
    "I32": (torch.int32, np.dtype("<i4"), 4),
    "I16": (torch.int16, np.dtype("<i2"), 2),
    "I8": (torch.int8, np.dtype("i1"), 1),
    "U8": (torch.uint8, np.dtype("u1"), 1),
    "BOOL": (torch.bool, np.dtype("u1"), 1),
}
_TAG_OF = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str                   # safetensors tag
    shape: Tuple[int, ...]
    begin: int                   # absolute file offsets
    end: int
    file: str

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype][0]


class SafetensorsFile:
    """One ``.safetensors`` file, memory-mapped; tensors are materialised on request."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        base = 8 + hlen
        self.metadata: Dict[str, str] = header.pop("__metadata__", {}) or {}
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            tag = info.get("dtype")
            if tag not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype '{tag}'")
            shape = tuple(int(s) for s in info.get("shape", []))
            b, e = info.get("data_offsets", [0, 0])
            nbytes = int(np.prod(shape, dtype=np.int64)) * _DTYPES[tag][2] if shape else _DTYPES[tag][2]
            if e - b != nbytes or base + e > size or b < 0:
                raise SafetensorsError(f"{path}: tensor '{name}' has data_offsets [{b}, {e}] that do not match "
                                       f"shape {list(shape)} of {tag} or the file size")
            self.entries[name] = TensorEntry(name, tag, shape, base + b, base + e, path)
        self._mm: Optional[mmap.mmap] = None

    def _map(self) -> mmap.mmap:
        if self._mm is None:
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        return self._mm

    def names(self) -> List[str]:
        return list(self.entries)

    def read(self, name: str) -> torch.Tensor:
        """A CPU tensor that owns its memory (copied out of the mapping)."""
        ent = self.entries[name]
        tdtype, ndtype, _ = _DTYPES[ent.dtype]
        count = int(np.prod(ent.shape, dtype=np.int64)) if ent.shape else 1
        arr = np.frombuffer(self._map(), dtype=ndtype, count=count, offset=ent.begin).copy()
        t = torch.from_numpy(arr)
        if ent.dtype == "BF16":
            t = t.view(torch.bfloat16)
        elif ent.dtype == "BOOL":
            t = t.to(torch.bool)
        return t.reshape(ent.shape)

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._f.close()


class TensorStore:
    """All tensors of a model folder: ``model.safetensors``, or the shards an index names."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        files = self._shard_files(model_dir)
        if not files:
            raise FileNotFoundError(f"{model_dir}: no model.safetensors (or *.safetensors shards)")
        self.files = [SafetensorsFile(p) for p in files]
        self.where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for n in f.entries:
                if n in self.where:
                    raise SafetensorsError(f"tensor '{n}' appears in both {self.where[n].path} and {f.path}")
                self.where[n] = f

    @staticmethod
    def _shard_files(model_dir: str) -> List[str]:
        single = os.path.join(model_dir, "model.safetensors")
        if os.path.isfile(single):
            return [single]
        index = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as f:
                weight_map = json.load(f).get("weight_map", {})
            names = sorted(set(weight_map.values()))
            paths = [os.path.join(model_dir, n) for n in names]
            missing = [p for p in paths if not os.path.isfile(p)]
            if missing:
                raise FileNotFoundError(f"{index} names shard files that do not exist: {', '.join(missing)}")
            return paths
        return sorted(os.path.join(model_dir, n) for n in os.listdir(model_dir) if n.endswith(".safetensors"))

    def names(self) -> List[str]:
        return list(self.where)

    def entry(self, name: str) -> TensorEntry:
        return self.where[name].entries[name]

    def read(self, name: str) -> torch.Tensor:
        return self.where[name].read(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write CPU tensors in name order.  Data is aligned to 8 bytes by padding the header."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    blobs: List[bytes] = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _TAG_OF:
            raise SafetensorsError(f"cannot store tensor '{name}' of dtype {t.dtype}")
        if t.dtype == torch.bfloat16:
            raw = t.view(torch.int16).numpy().tobytes()
        elif t.dtype == torch.bool:
            raw = t.to(torch.uint8).numpy().tobytes()
        else:
            raw = t.numpy().tobytes()
        header[name] = {"dtype": _TAG_OF[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hbytes = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hbytes += b" " * ((8 - len(hbytes) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hbytes)))
        f.write(hbytes)
        for raw in blobs:
            f.write(raw)
