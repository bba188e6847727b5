"""Architectures the package knows; importing this module registers them."""

from . import qwen3  # noqa: F401
