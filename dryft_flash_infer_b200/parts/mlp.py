"""The dense SwiGLU feed-forward."""

from __future__ import annotations

from ..ops import kernels
from .base import FeedForward, TensorDecl, register_part


class SwiGLU(FeedForward):
    """``down(silu(gate(x)) * up(x))`` without biases; gate and up share one fused matrix
    ``[2*inter, hidden]`` with the gate rows first (engine/engine.py:173-176;
    engine/kernels/reference.py:74-79)."""

    kind = "swiglu"
    accepts_scaled_rows = True
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu"):
        if activation != "silu":
            raise ValueError(f"SwiGLU feed-forward knows the 'silu' activation only, got {activation!r}")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.gate_up = self.down = None

    @property
    def fuses_add_norm(self) -> bool:
        # the product that would add and prepare the next norm is the down projection, whose inner size is the
        # intermediate one: the decode kernel takes it in steps of 8 (other sizes run the plain kernels)
        return self.intermediate_size % 8 == 0

    def tensors(self):
        inter, hidden = self.intermediate_size, self.hidden_size
        return {
            "gate_proj": TensorDecl((inter, hidden), "gate_up", 0),
            "up_proj": TensorDecl((inter, hidden), "gate_up", inter),
            "down_proj": TensorDecl((hidden, inter), "down"),
        }

    def first_weights(self):
        return kernels.next_weights(self.gate_up, swiglu=True)

    def forward(self, x, ctx, add_norm=None):
        inner = kernels.linear_swiglu(x, self.gate_up, then=kernels.next_weights(self.down))
        return kernels.linear(inner, self.down, add_norm=add_norm, then=getattr(ctx, "upcoming", None))


register_part("feed_forward", SwiGLU.kind, SwiGLU)
