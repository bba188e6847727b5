"""A model described as data: which parts each layer has, and in which order layers run.

An architecture's builder (see ``models/``) turns a typed configuration into a
``ModelSpec``.  Everything downstream (weight loading, cache layout, the step
function) works from the spec and never asks which architecture it came from.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: its registered kind and the parameters of its constructor."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement (``block``) of a mixer, a feed-forward and their norms.

    ``tensor_names`` maps each tensor of the layer, written ``<part>.<tensor>`` with
    part in {mixer, feed_forward, mixer_norm, ffn_norm}, to its name in the model file.
    """

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    ffn_norm: PartSpec
    tensor_names: dict[str, str]


@dataclass(frozen=True)
class ScheduleEntry:
    """One application of a layer.

    ``layer`` indexes ``ModelSpec.layers`` and may occur in several entries (the
    same weights run twice).  ``cache`` is the cache entry this application
    attends over; entries that own their cache have a number of their own, and an
    entry with ``writes_cache=False`` reads what an earlier entry of the same
    step wrote under that number.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    embedding_name: str
    final_norm_names: dict[str, str]
    #: name of the output head's matrix, or None when it is the embedding table
    head_name: str | None

    def check(self) -> None:
        owners = {}
        for position, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule[{position}] names layer {entry.layer}, model has {len(self.layers)}")
            if entry.writes_cache:
                if entry.cache in owners:
                    raise ValueError(f"schedule[{position}]: cache {entry.cache} already written by "
                                     f"schedule[{owners[entry.cache]}]")
                owners[entry.cache] = position
            elif entry.cache not in owners:
                raise ValueError(f"schedule[{position}] reads cache {entry.cache} before any entry wrote it")


def straight_schedule(n_layers: int) -> tuple[ScheduleEntry, ...]:
    """Every layer once, in order, each with a cache of its own."""
    return tuple(ScheduleEntry(layer=i, cache=i) for i in range(n_layers))
