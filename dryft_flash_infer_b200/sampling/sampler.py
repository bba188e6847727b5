"""Choosing the next token: greedy, or at a temperature with a reproducible random number.

The reference only takes the argmax (engine/engine.py:1026, :1046).  Temperature
sampling draws from ``softmax(logits / temperature)`` by inverse CDF at a uniform number
that depends on (seed, request, step) alone, so what a request generates does not depend
on which batch it runs in or where it stands in that batch.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..ops import kernels

_MASK = (1 << 64) - 1


def _mix(x: int) -> int:
    """The splitmix64 finaliser."""
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform_for(seed: int, request: int, step: int) -> float:
    """A number in [0, 1) with 24 random bits, fixed by (seed, request, step)."""
    h = _mix(_mix(_mix(seed & _MASK) ^ (request & _MASK)) ^ (step & _MASK))
    return (h >> 40) / float(1 << 24)


@dataclass(frozen=True)
class SamplingParams:
    """``temperature`` 0 means greedy (argmax, lowest index on ties)."""

    temperature: float = 0.0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")


def select_tokens(logits: torch.Tensor, params: SamplingParams, requests: list[int], step: int) -> torch.Tensor:
    """Next token for each row of float32 ``logits`` on the device (int32 tensor, on the device)."""
    if params.temperature == 0.0:
        return kernels.argmax(logits)
    u = np.array([uniform_for(params.seed, r, step) for r in requests], dtype=np.float32)
    uniforms = torch.from_numpy(u).to(logits.device)
    return kernels.sample_temperature(logits, uniforms, params.temperature)
