"""Rotary position embedding: the angle tables that an attention mixer rotates q and k by."""

from __future__ import annotations

import torch

from .base import PositionEncoding, register_part


class RotaryEmbedding(PositionEncoding):
    """Half-split rotary embedding with absolute positions.

    ``inv_freq_i = theta^(-i / (D/2))`` for ``i < D/2``; the angle of position ``p`` is
    ``p * inv_freq_i`` for the pair ``(i, i + D/2)``, all in float32
    (engine/engine.py:350-356).  The tables are ``[max_positions, D/2]`` float32 and stay
    float32 in the bfloat16 engine too (the reference rounds them to bfloat16, :357-358).
    """

    kind = "rotary"
    graph_safe = True

    def __init__(self, hidden_size: int, head_dim: int, theta: float):
        if head_dim % 2:
            raise ValueError(f"rotary embedding needs an even head_dim, got {head_dim}")
        self.head_dim, self.theta = head_dim, float(theta)
        self.cos = self.sin = None

    def prepare(self, max_positions: int, device) -> None:
        half = self.head_dim // 2
        steps = torch.arange(0, half, dtype=torch.int64).float()
        inv_freq = 1.0 / (self.theta ** (steps / half))
        positions = torch.arange(max_positions, dtype=torch.int64).float()
        angles = positions[:, None] * inv_freq[None, :]
        self.cos = angles.cos().contiguous().to(device)
        self.sin = angles.sin().contiguous().to(device)


register_part("position", RotaryEmbedding.kind, RotaryEmbedding)
