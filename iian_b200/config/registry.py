"""One registry from an architecture's name (``config.json``'s ``architectures[0]``) to the
plug-in that knows it.

Mirrors the reference's ``ArchRegistry`` / ``IIAN_REGISTER_ARCH`` (include/iian/arch.h:36-52,
src/iian/model_loader.cpp:536-546): a plug-in registers itself when its module is imported,
and an unknown name is an error that lists the names that are known
(src/iian/model_loader.cpp:315-319).
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Mapping, Type


class Architecture:
    """What an architecture has to provide.

    * ``name``: the string in ``config.json``'s ``architectures`` list.
    * ``load_config(dict) -> config``: typed configuration from the file's own keys
      (the reference's ``load_hparams``).
    * ``build_spec(config) -> ModelSpec``: parts per layer and the run order
      (the reference's ``build_graph``, as data).
    * ``tensor_name(scope, local) -> str``: the name in the weight file of a part's tensor
      (the reference's ``create_tensors`` naming).  ``scope`` is ``("embedding",)``,
      ``("final_norm",)``, ``("head",)`` or ``("layer", i, slot)`` with ``slot`` one of
      ``mixer``, ``feed_forward``, ``mixer_norm``, ``feed_forward_norm``.
    * ``config_to_dict(config) -> dict``: the ``config.json`` content for a configuration
      (used by the random-weights writer).
    """

    name: str = ""

    def load_config(self, raw: Mapping[str, Any]):  # pragma: no cover - interface
        raise NotImplementedError

    def build_spec(self, config):  # pragma: no cover - interface
        raise NotImplementedError

    def tensor_name(self, scope: tuple, local: str) -> str:  # pragma: no cover - interface
        raise NotImplementedError

    def config_to_dict(self, config) -> Dict[str, Any]:  # pragma: no cover - interface
        raise NotImplementedError


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(cls: Type[Architecture]) -> Type[Architecture]:
    """Class decorator: instantiate and register under ``cls.name``."""
    inst = cls()
    if not inst.name:
        raise ValueError(f"{cls.__name__} has no name")
    _ARCHITECTURES[inst.name] = inst
    return cls


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def architecture_names() -> list[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _load_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise KeyError(f"unknown architecture '{name}'; supported: {', '.join(sorted(_ARCHITECTURES))}") from None


def _load_builtin() -> None:
    # importing the module registers the plug-in
    from ..models import qwen3  # noqa: F401


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{model_dir}: no config.json")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    if not isinstance(raw, dict):
        raise ValueError(f"{path}: expected a JSON object")
    return raw


def architecture_of(raw: Mapping[str, Any]) -> Architecture:
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ValueError("config.json: 'architectures' must be a non-empty list of names")
    return get_architecture(archs[0])


def load_model_config(model_dir: str):
    """``(architecture, typed config)`` for a model folder."""
    raw = read_config_json(model_dir)
    arch = architecture_of(raw)
    return arch, arch.load_config(raw)
