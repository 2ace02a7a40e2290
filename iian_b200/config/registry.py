"""One registry from an architecture's name (``config.json``'s ``architectures[0]``, or its ``architecture``) to the
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
    # True: some sizes are given by the shapes of the weight file's tensors only; ``with_tensor_sizes(raw, shapes)`` then
    # returns ``raw`` completed with them before ``load_config`` sees it (``load_model_config``)
    reads_tensor_shapes: bool = False

    def with_tensor_sizes(self, raw: Mapping[str, Any], shapes: Mapping[str, tuple]) -> Mapping[str, Any]:
        return raw

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
    from ..models import galodra, lekilix, nogelorn, qwen3, senadra  # noqa: F401


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
    """The plug-in a ``config.json`` names: the first entry of ``architectures`` (a list of names), or ``architecture``
    (one name)."""
    archs = raw.get("architectures")
    if archs is None and isinstance(raw.get("architecture"), str):
        archs = [raw["architecture"]]
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ValueError("config.json: 'architectures' must be a non-empty list of names (or 'architecture' one name)")
    return get_architecture(archs[0])


def load_model_config(model_dir: str):
    """``(architecture, typed config)`` for a model folder."""
    raw = read_config_json(model_dir)
    arch = architecture_of(raw)
    if arch.reads_tensor_shapes:
        raw = arch.with_tensor_sizes(raw, tensor_shapes(model_dir))
    return arch, arch.load_config(raw)


def tensor_shapes(model_dir: str) -> Dict[str, tuple]:
    """Name -> shape of every tensor in the folder's weight file(s); only the headers are read.  Empty without a file."""
    from ..weights.safetensors_io import SafetensorsError, TensorStore
    try:
        store = TensorStore(model_dir)
    except (FileNotFoundError, SafetensorsError):
        return {}
    try:
        return {name: tuple(store.entry(name).shape) for name in store.names()}
    finally:
        store.close()
