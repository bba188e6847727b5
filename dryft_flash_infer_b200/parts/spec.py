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
    """One layer: the arrangement (``block``) of a mixer, a feed-forward and the block's norms.

    ``norms`` maps the names the block kind gives its norms to their specs: the block
    decides how many it has and where they stand (``pre_norm`` has ``mixer_norm`` and
    ``ffn_norm``).  ``tensor_names`` maps each tensor of the layer, written
    ``<part>.<tensor>`` with part in {mixer, feed_forward} or a norm's name, to its name
    in the model file.
    """

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: dict[str, PartSpec]
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
    #: the norm between the last block and the output head, or None for a model without one
    final_norm: PartSpec | None
    embedding_name: str
    final_norm_names: dict[str, str]
    #: name of the output head's matrix, or None when it is the embedding table
    head_name: str | None
    #: what surrounds the blocks, for architectures that have it: a factor on the embedded rows, a
    #: factor on the logits, and a cap ``c`` that turns logits ``x`` into ``c * tanh(x / c)`` (0: none)
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    logit_softcap: float = 0.0
    #: tensors that a model file may hold beside the expected ones without being an error
    ignorable_tensors: tuple[str, ...] = ()

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
