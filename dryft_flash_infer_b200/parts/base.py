"""Interfaces of the parts a layer is made of, and the registries that hold their kinds.

A part is built from its own parameters only (sizes, constants); it does not know
which model it is in.  It declares its tensors by a local name; the
architecture's builder maps local names to names in the model file.

Interfaces
----------
Norm          ``forward(x) -> normed``; ``add_forward(residual, delta) -> normed``
              (adds ``delta`` into ``residual`` in place first).
Position      ``prepare(max_positions, device)``; what the mixer reads from it is
              between the two of them (rotary: ``cos``/``sin`` tables).
Mixer         ``cache_need()``, ``state_need()``, ``forward(x, ctx, cache, state)``.
FeedForward   ``forward(x, ctx)``.
Block         ``norm_names``; ``forward(residual, pending, ctx, cache, state) -> (residual, pending)``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

from .spec import PartSpec


@dataclass(frozen=True)
class TensorDecl:
    """One tensor a part wants from the model file.

    It lands in rows ``row_start ...`` of the part's device buffer ``buffer``, so
    that several file tensors can share one fused matrix without a second copy.
    ``init`` picks the random-weights rule: ``matrix`` or ``norm``.  ``precision``
    is ``compute`` (held in the engine's dtype) or ``float32`` (always 32-bit).
    """

    shape: tuple[int, ...]
    buffer: str
    row_start: int = 0
    init: str = "matrix"
    precision: str = "compute"


@dataclass(frozen=True)
class KVNeed:
    """A mixer that keeps keys and values per token: heads, head size and, if not 0,
    the window of latest tokens that it ever reads."""

    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps a state of fixed size per sequence: its shape, the dtype it is held in
    (``float32`` or ``bfloat16``) and the value every element has when a sequence starts."""

    shape: tuple[int, ...]
    dtype: str = "float32"
    init: float = 0.0


class Part:
    kind = ""
    #: True if the part's ``forward`` only launches work on the current stream from device-resident
    #: numbers (no host read-back, no shape that depends on values), so that a decode step through
    #: it can be captured in a CUDA graph.  A model decodes through a graph only if all its parts say so.
    graph_safe = False
    #: True if ``forward`` takes its rows as ``kernels.ScaledRows`` too (normalised rows that may still
    #: lack their 1/rms factor, which the part's first product applies: it hands them to
    #: ``kernels.linear`` as they are)
    accepts_scaled_rows = False
    #: True if ``forward`` takes ``add_norm=(residual, weight, eps)``: its last product then adds its
    #: result to ``residual`` in place and returns the ``ScaledRows`` of the norm that follows
    fuses_add_norm = False

    def tensors(self) -> dict[str, TensorDecl]:
        return {}

    def bind(self, buffers: dict[str, torch.Tensor]) -> None:
        """Receives the device buffers named in ``tensors()`` once they are filled."""
        for name, tensor in buffers.items():
            setattr(self, name, tensor)

    def first_weights(self):
        """``kernels.NextWeights`` of the matrix that ``forward`` streams first, or None.  Whoever runs
        this part after another one may leave it in ``ctx.upcoming``, where the part before finds it and
        hands it to its last kernel (``then=``): a hint for decode steps that changes no result."""
        return None

    def buffer_shapes(self) -> dict[str, tuple[tuple[int, ...], str]]:
        out: dict[str, tuple[tuple[int, ...], str]] = {}
        for decl in self.tensors().values():
            rows = decl.row_start + decl.shape[0]
            shape, precision = out.get(decl.buffer, ((0,) + decl.shape[1:], decl.precision))
            if shape[1:] != decl.shape[1:] or precision != decl.precision:
                raise ValueError(f"tensors sharing buffer '{decl.buffer}' disagree on shape or precision")
            out[decl.buffer] = ((max(shape[0], rows),) + decl.shape[1:], precision)
        return out


class Norm(Part):
    def forward(self, x):
        raise NotImplementedError

    def add_forward(self, residual, delta):
        residual.add_(delta)
        return self.forward(residual)

    def scale_fusion(self):
        """``(weight, eps)`` if the norm is ``x / rms(x) * weight`` over the whole row, so that a product
        before it can prepare it and the product after it can finish it; else None."""
        return None


class PositionEncoding(Part):
    def prepare(self, max_positions: int, device) -> None:
        pass


class Mixer(Part):
    def cache_need(self) -> KVNeed | None:
        return None

    def state_need(self) -> StateNeed | None:
        return None

    def prepare(self, max_positions: int, device) -> None:
        pass

    def forward(self, x, ctx, cache, state):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx):
        raise NotImplementedError


class Block:
    """An arrangement of a mixer, a feed-forward and norms around the residual stream.  How many norms
    there are and where they stand is the block kind's business: it names them in ``norm_names``.

    The residual stream travels between blocks as ``(residual, pending)``: ``pending``
    is a delta not yet added, so that the next norm can add and normalise in one pass.
    """

    kind = ""
    #: True if ``forward`` takes ``next_norm`` (the norm that will read this block's result) and may
    #: then return ``pending`` as ``kernels.ScaledRows`` of that norm, the sum already in ``residual``
    fuses_next_norm = False

    #: the names of the norms this arrangement has; the layer's spec must give exactly these
    norm_names: tuple[str, ...] = ()

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: dict[str, Norm]):
        if set(norms) != set(self.norm_names):
            raise ValueError(f"a '{self.kind}' block has the norms {sorted(self.norm_names)}, the layer gives "
                             f"{sorted(norms)}")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.norms = dict(norms)

    def parts(self) -> dict[str, Part]:
        return {"mixer": self.mixer, "feed_forward": self.feed_forward, **self.norms}

    @property
    def first_norm(self) -> Norm | None:
        """The norm that reads the residual stream as it enters the block, if the block starts with one."""
        return None

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part in self.parts().values())

    @property
    def takes_scaled_pending(self) -> bool:
        """True if ``pending`` may arrive as ``ScaledRows`` of this block's first norm."""
        return False

    def forward(self, residual, pending, ctx, cache, state):
        raise NotImplementedError


_REGISTRIES: dict[str, dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {},
}


def register_part(category: str, kind: str, factory: Callable) -> None:
    """Registers ``factory(hidden_size=..., **params)`` (for blocks: the class) under ``kind``."""
    if category not in _REGISTRIES:
        raise ValueError(f"unknown part category '{category}'; known: {', '.join(_REGISTRIES)}")
    _REGISTRIES[category][kind] = factory


def part_factory(category: str, kind: str) -> Callable:
    table = _REGISTRIES[category]
    if kind not in table:
        raise ValueError(f"unknown {category} kind '{kind}'; known: {', '.join(sorted(table)) or 'none'}")
    return table[kind]


def build_part(category: str, spec: PartSpec, hidden_size: int):
    return part_factory(category, spec.kind)(hidden_size=hidden_size, **spec.params)
