"""The one registry from an architecture's name to its configuration class.

config.json names the architecture in `architectures`; the class registered
under that name parses the rest of the file and produces the `ModelPlan`.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Type

_ARCHITECTURES: Dict[str, Type] = {}


class ConfigError(ValueError):
    """A config.json that cannot be used: missing key, wrong type, unsupported option."""


def register_architecture(name: str, config_class: Type) -> None:
    """`config_class` needs `from_dict(dict)`, `to_dict()` and `plan()`."""
    for attr in ("from_dict", "to_dict", "plan"):
        if not hasattr(config_class, attr):
            raise TypeError(f"configuration class for {name!r} lacks {attr}()")
    _ARCHITECTURES[name] = config_class


def known_architectures():
    return sorted(_ARCHITECTURES)


def config_class_for(name: str) -> Type:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture {name!r}; known: {known_architectures()}") from None


def config_from_dict(root: dict, **options):
    """Choose the configuration class by `architectures` and let it parse `root`
    (`options` go to its `from_dict`, e.g. `strict=True`)."""
    if not isinstance(root, dict):
        raise ConfigError("model config root must be a JSON object")
    if "architectures" not in root:
        raise ConfigError("missing required config field 'architectures'")
    names = root["architectures"]
    if not isinstance(names, list):
        raise ConfigError("config field 'architectures' must be an array")
    for name in names:
        if isinstance(name, str) and name in _ARCHITECTURES:
            return _ARCHITECTURES[name].from_dict(root, **options) if options else _ARCHITECTURES[name].from_dict(root)
    raise ConfigError(f"no supported architecture in {names!r}; known: {known_architectures()}")


def load_config(path: str):
    """Read `path` (a model folder or a config.json) through the registry."""
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            root = json.load(f)
    except OSError as e:
        raise ConfigError(f"cannot open model config: {path}: {e}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"cannot parse model config {path!r}: {e}") from None
    return config_from_dict(root)
