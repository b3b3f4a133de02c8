"""One registry from an architecture's name to its configuration class.

``config.json``'s ``architectures[0]`` picks the entry; the entry's class reads
the architecture's own keys and turns them into a ``ModelSpec``.  NNIS has a
hard check in place of a table (crates/nnis-model/src/safetensors_loader.rs:137-145);
an unknown name fails here with the known names in the message.

Adding an architecture = one configuration class with ``from_dict``,
``to_dict`` and ``to_spec`` and one ``register_architecture`` call.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Mapping, Type

from .llama import ConfigError, LlamaConfig
from .spec import ModelSpec

_ARCHITECTURES: Dict[str, Type] = {}


def register_architecture(name: str, config_cls: Type) -> None:
    for attr in ("from_dict", "to_dict", "to_spec"):
        if not hasattr(config_cls, attr):
            raise TypeError(f"{config_cls.__name__} lacks {attr}()")
    _ARCHITECTURES[name] = config_cls


def known_architectures():
    return sorted(_ARCHITECTURES)


def config_from_dict(raw: Mapping[str, Any]):
    archs = raw.get("architectures")
    if not isinstance(archs, list) or len(archs) != 1 or not isinstance(archs[0], str):
        raise ConfigError(f"config.json: architectures must be a list of one name; got {archs!r}")
    cls = _ARCHITECTURES.get(archs[0])
    if cls is None:
        raise ConfigError(f"config.json: unknown architecture {archs[0]!r}; "
                          f"known: {known_architectures()}")
    return cls.from_dict(raw)


def read_config(model_dir: str):
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        # NNIS's own folder carries its configuration in model.json
        from ..weights.nnis_directory import (NnisDirectoryError, config_of_manifest, is_nnis_directory,
                                              read_manifest)
        if is_nnis_directory(model_dir):
            try:
                return config_from_dict(config_of_manifest(read_manifest(model_dir)))
            except NnisDirectoryError as e:
                raise ConfigError(str(e)) from None
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON: {e}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: the top level must be an object")
    return config_from_dict(raw)


def spec_from_dir(model_dir: str) -> ModelSpec:
    return read_config(model_dir).to_spec()


register_architecture(LlamaConfig.architecture, LlamaConfig)
