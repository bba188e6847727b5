"""Fills a model's device buffers from a model folder, by tensor name.

Matrices are held in the engine's dtype (bfloat16 in serving: a bfloat16 or float16
tensor of the file is taken as is or converted, a float32 one is rounded); tensors that
a part declares ``float32`` (norm weights) are held in float32 whatever the file stores,
so a tensor stored in 32-bit loses nothing.  Integer tensors would be held as int32.
Everything that is wrong with the file's tensors is reported in one error.
"""

from __future__ import annotations

from pathlib import Path

import torch

from .safetensors_io import ModelFiles, SafetensorsError

_FLOATS = (torch.float32, torch.bfloat16, torch.float16)


class WeightError(ValueError):
    """The model file does not fit the architecture.  ``missing``, ``unexpected``,
    ``wrong_shape`` (name, found, wanted) and ``wrong_dtype`` list every tensor at fault."""

    def __init__(self, folder, missing, unexpected, wrong_shape, wrong_dtype):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = [f"weights in {folder} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, found, wanted in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(found)}, expected {list(wanted)}")
        for name, found in self.wrong_dtype:
            lines.append(f"  unsupported dtype: {name} is {found}")
        super().__init__("\n".join(lines))


def check_tensors(folder, files: ModelFiles, expected, ignorable=()) -> None:
    wanted = {e.name: e for e in expected}
    present = set(files.names())
    missing = [n for n in wanted if n not in present]
    unexpected = sorted(n for n in present if n not in wanted and n not in ignorable)
    wrong_shape, wrong_dtype = [], []
    for name, e in wanted.items():
        if name in present:
            dtype, shape = files.info(name)
            if tuple(shape) != tuple(e.decl.shape):
                wrong_shape.append((name, shape, e.decl.shape))
            if dtype not in _FLOATS:
                wrong_dtype.append((name, dtype))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(folder, missing, unexpected, wrong_shape, wrong_dtype)


def load_weights(model, folder: str | Path) -> None:
    """Copies every expected tensor from ``folder`` into ``model``'s allocated buffers."""
    files = ModelFiles(folder)
    expected = model.expected_tensors()
    # a tied model's file may still carry a copy of the head: it is the embedding, so it is skipped
    ignorable = ("lm_head.weight",) if model.spec.head_name is None else ()
    check_tensors(folder, files, expected, ignorable)
    for e in expected:
        model.destination(e).copy_(files.tensor(e.name))
    model.bind()


__all__ = ["WeightError", "SafetensorsError", "check_tensors", "load_weights"]
