"""The hand-written CUDA operations of the engine (see ``kernels.py``) and their build."""

from . import kernels
from .build import BuildError
from .kernels import KernelError

__all__ = ["kernels", "BuildError", "KernelError"]
