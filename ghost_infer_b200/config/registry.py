"""One registry from an architecture's name (config.json `architectures[0]`) to its model.

The reference has no registry object: a constant list of GGUF architecture
names gates loading (src/model.rs:135, src/model.rs:139-142) and one struct
switches on enum variants per layer (src/model.rs:336-362).  Here an
architecture is two functions: one that types its config.json and one that
turns the typed configuration into a `ModelSpec` (a list of layers put
together from parts, plus the order in which they run).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from .errors import ConfigError, UnknownArchitectureError


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], Any]
    build_spec: Callable[[Any], Any]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config: Callable[[Mapping[str, Any]], Any],
                          build_spec: Callable[[Any], Any], *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture \"{name}\" is already registered")
    _ARCHITECTURES[name] = Architecture(name, parse_config, build_spec)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> tuple:
    return tuple(sorted(_ARCHITECTURES))


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise UnknownArchitectureError(
            f"architecture \"{name}\" is not supported (registered: {', '.join(registered_architectures()) or 'none'})"
        ) from None


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: the top level must be an object")
    return raw


def architecture_of(raw: Mapping[str, Any]) -> str:
    archs = raw.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: \"architectures\" must be a non-empty list of names")
    return archs[0]


def parse_config(raw: Mapping[str, Any]):
    """Typed configuration of whatever architecture `raw` names."""
    return get_architecture(architecture_of(raw)).parse_config(raw)


def load_config(model_dir: str):
    return parse_config(read_config_json(model_dir))
