"""One registry from the architecture's name (config.json ``architectures[0]``) to
its model.  The reference has none: it never looks at ``architectures`` and runs
any checkpoint with the right tensor names (cmd/gollmgo/gpu.go:91-92).

An architecture is two functions: ``parse(config_dict) -> typed config`` and
``spec(typed config) -> ModelSpec`` (gollmgo_b200/parts/spec.py).  Everything below
the spec is generic.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict

from .model_config import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    parse: Callable      # dict -> typed config
    spec: Callable       # typed config -> parts.spec.ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse: Callable, spec: Callable) -> None:
    _ARCHITECTURES[name] = Architecture(name, parse, spec)


def known_architectures():
    return sorted(_ARCHITECTURES)


def resolve_architecture(config_dict: dict) -> Architecture:
    archs = config_dict.get("architectures")
    if not archs:
        raise ConfigError("config.json: 'architectures' is missing; known: "
                          + ", ".join(known_architectures()))
    for a in archs:
        if a in _ARCHITECTURES:
            return _ARCHITECTURES[a]
    raise ConfigError(f"config.json: architecture {list(archs)} is not registered; known: "
                      + ", ".join(known_architectures()))
