"""The one registry from an architecture's name to what builds it.

``config.json`` names its architecture (``architectures[0]``, else ``model_type``);
the registry maps that name to the typed configuration class, whose
``model_spec()`` lists the parts of every layer.  The reference has one
hard-wired model (src/transformer.cpp:44-99) and no names.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Type

from .spec import ConfigError

_ARCHITECTURES: Dict[str, Type] = {}


def register_architecture(name: str, config_class: Type) -> None:
    """``config_class`` needs ``from_dict(dict)``, ``to_dict()`` and ``model_spec()``."""
    _ARCHITECTURES[name] = config_class


def known_architectures():
    return sorted(_ARCHITECTURES)


def architecture_name(d: Dict[str, Any]) -> str:
    name = (d.get("architectures") or [None])[0] or d.get("model_type")
    if not name:
        raise ConfigError("config.json names no architecture ('architectures' or 'model_type'); "
                          f"known: {known_architectures()}")
    return str(name)


def config_from_dict(d: Dict[str, Any]):
    name = architecture_name(d)
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture {name!r}; known: {known_architectures()}")
    return _ARCHITECTURES[name].from_dict(d)


def load_config(folder: str):
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path} does not exist")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path} is not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return config_from_dict(d)
