"""One registry from the architecture's name (``config.json["architectures"][0]``) to its
configuration class. The reference maps ``architecture=...`` in config.ini to flags the
same way and refuses unknown names (src/config.c:83-87)."""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Mapping

from .spec import ConfigError

_ARCHITECTURES: Dict[str, Callable[[Mapping[str, Any]], Any]] = {}


def register_architecture(name: str, config_class: Callable[[Mapping[str, Any]], Any]) -> None:
    """``config_class.from_json(raw)`` must return an object with ``model_spec()`` and
    ``to_json()``. Registering a name twice replaces the entry (tests register toys)."""
    _ARCHITECTURES[name] = config_class


def architectures() -> Dict[str, Any]:
    return dict(_ARCHITECTURES)


def config_from_json(raw: Mapping[str, Any]):
    """Chooses the configuration class by the architecture's name and parses ``raw``."""
    names = raw.get("architectures")
    if not isinstance(names, (list, tuple)) or not names or not isinstance(names[0], str):
        raise ConfigError("config.json: missing required key(s): architectures")
    name = names[0]
    if name not in _ARCHITECTURES:
        known = ", ".join(sorted(_ARCHITECTURES)) or "none"
        raise ConfigError(f"unsupported architecture: {name} (known: {known})")
    return _ARCHITECTURES[name].from_json(raw)


def load_config(model_dir: str):
    """Reads ``<model_dir>/config.json``."""
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: must hold a JSON object")
    return config_from_json(raw)
