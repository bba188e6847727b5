"""Rotary position embedding: the angle tables that an attention mixer rotates q and k by."""

from __future__ import annotations

import torch

from .base import PositionEncoding, register_part


class RotaryEmbedding(PositionEncoding):
    """Half-split rotary embedding with absolute positions.

    ``inv_freq_i = theta^(-i / (r/2))`` for ``i < r/2``; the angle of position ``p`` is
    ``p * inv_freq_i`` for the pair ``(i, i + r/2)``, all in float32
    (engine/engine.py:350-356), where ``r = rotary_dim`` is the number of elements of a head
    that rotate: the whole head by default, as in the reference, or only its first ``r``.
    The tables are ``[max_positions, r/2]`` float32 and stay float32 in the bfloat16 engine
    too (the reference rounds them to bfloat16, :357-358).
    """

    kind = "rotary"
    graph_safe = True

    def __init__(self, hidden_size: int, head_dim: int, theta: float, rotary_dim: int | None = None):
        rotary_dim = head_dim if rotary_dim is None else int(rotary_dim)
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary embedding rotates an even number of elements, at most head_dim = {head_dim}; "
                             f"got {rotary_dim}")
        self.head_dim, self.rotary_dim, self.theta = head_dim, rotary_dim, float(theta)
        self.cos = self.sin = None

    def prepare(self, max_positions: int, device) -> None:
        half = self.rotary_dim // 2
        steps = torch.arange(0, half, dtype=torch.int64).float()
        inv_freq = 1.0 / (self.theta ** (steps / half))
        positions = torch.arange(max_positions, dtype=torch.int64).float()
        angles = positions[:, None] * inv_freq[None, :]
        self.cos = angles.cos().contiguous().to(device)
        self.sin = angles.sin().contiguous().to(device)


register_part("position", RotaryEmbedding.kind, RotaryEmbedding)
