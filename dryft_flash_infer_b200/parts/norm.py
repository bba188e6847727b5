"""RMSNorm, alone and with the residual add fused in front of it."""

from __future__ import annotations

from ..ops import kernels
from .base import Norm, TensorDecl, register_part


class RMSNorm(Norm):
    """``x * rsqrt(mean(x^2) + eps) * weight`` (engine/kernels/reference.py:13-16).

    ``add_forward`` is the reference's ``add_rms_norm`` (reference.py:19-23): the sum is
    written back as the new residual and normalised in the same pass.  The weight is
    held in float32 whatever the engine's dtype.
    """

    kind = "rms_norm"
    graph_safe = True

    def __init__(self, hidden_size: int, eps: float, dim: int | None = None):
        self.dim = dim if dim is not None else hidden_size
        self.eps = float(eps)
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.dim,), "weight", init="norm", precision="float32")}

    def forward(self, x):
        return kernels.rms_norm(x, self.weight, self.eps)

    def add_forward(self, residual, delta):
        return kernels.add_rms_norm(residual, delta, self.weight, self.eps)

    def scale_fusion(self):
        return self.weight, self.eps


register_part("norm", RMSNorm.kind, RMSNorm)
