"""Typed model configurations read from a model folder's ``config.json``."""

from __future__ import annotations

import json
from dataclasses import dataclass, fields
from pathlib import Path
from typing import Any, ClassVar


class ConfigError(ValueError):
    """A ``config.json`` that cannot be used: the message names the key."""


_MISSING = object()


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration.

    A subclass lists the keys of its architecture's ``config.json`` as dataclass
    fields and checks them in ``validate``.  Nothing else in the package holds a
    size or a constant that ``config.json`` gives.
    """

    architecture: ClassVar[str] = ""
    #: the checkpoint format's ``model_type`` key, written beside ``architectures`` by ``save``
    model_type: ClassVar[str] = ""

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict[str, Any]:
        out = {"architectures": [self.architecture]}
        if self.model_type:
            out["model_type"] = self.model_type
        for f in fields(self):
            out[f.name] = getattr(self, f.name)
        return out

    def save(self, folder: str | Path) -> None:
        Path(folder).mkdir(parents=True, exist_ok=True)
        with open(Path(folder) / "config.json", "w") as fh:
            json.dump(self.to_dict(), fh, indent=2)


def take(raw: dict, key: str, kind, default=_MISSING):
    """``raw[key]`` checked to be of ``kind`` (int, float, bool, str)."""
    if key not in raw or raw[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: missing key '{key}'")
        return default
    value = raw[key]
    if kind is float and isinstance(value, (int, float)) and not isinstance(value, bool):
        return float(value)
    if kind is int and (isinstance(value, bool) or not isinstance(value, int)):
        raise ConfigError(f"config.json: '{key}' must be an integer, got {value!r}")
    if not isinstance(value, kind):
        raise ConfigError(f"config.json: '{key}' must be {kind.__name__}, got {value!r}")
    return value


def read_config_json(folder: str | Path) -> dict[str, Any]:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"no config.json in {folder}")
    try:
        with open(path) as fh:
            raw = json.load(fh)
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON ({exc})") from exc
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return raw
