"""One registry from an architecture's name to its configuration class and model builder."""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Callable

from .base import ConfigError, ModelConfig, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    #: ``build(config) -> ModelSpec``: the layers, their order and their tensor names.
    build: Callable


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build: Callable) -> None:
    """Adds (or replaces) the architecture called ``name`` in ``config.json``'s ``architectures``."""
    _ARCHITECTURES[name] = Architecture(name, config_class, build)


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_named(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture '{name}'; known: {', '.join(known_architectures()) or 'none'}")
    return _ARCHITECTURES[name]


def architecture_of(raw: dict) -> Architecture:
    names = raw.get("architectures")
    if not isinstance(names, list) or not names or not isinstance(names[0], str):
        raise ConfigError("config.json: 'architectures' must be a list holding the model class name")
    return architecture_named(names[0])


def config_from_dict(raw: dict) -> ModelConfig:
    return architecture_of(raw).config_class.from_dict(raw)


def load_config(folder: str | Path) -> ModelConfig:
    """The typed configuration of the model in ``folder``, chosen by ``architectures[0]``."""
    return config_from_dict(read_config_json(folder))
