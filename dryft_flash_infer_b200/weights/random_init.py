"""Random weights from a configuration and a seed: into a model folder, or straight onto the device.

Matrices are N(0, 0.02) and norm weights 1 + N(0, 0.01).  Every tensor has its own
generator seeded from (seed, tensor name), so a tensor's values do not depend on which
other tensors the model has or on the order they are made in.
"""

from __future__ import annotations

import hashlib
from pathlib import Path

import torch

from ..config import ModelConfig, architecture_named
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.01


def _tensor_seed(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:7], "little")


def random_tensor(name: str, shape, init: str, seed: int, device="cpu") -> torch.Tensor:
    """Float32 values of tensor ``name`` under ``seed``; ``init`` is ``matrix`` or ``norm``."""
    g = torch.Generator(device=device).manual_seed(_tensor_seed(seed, name))
    noise = torch.randn(tuple(shape), generator=g, device=device, dtype=torch.float32)
    if init == "norm":
        return 1.0 + NORM_STD * noise
    if init == "matrix":
        return MATRIX_STD * noise
    raise ValueError(f"unknown init rule '{init}'")


def fill_random(model, seed: int) -> None:
    """Fills ``model``'s allocated device buffers with random weights made on its device."""
    for e in model.expected_tensors():
        model.destination(e).copy_(random_tensor(e.name, e.decl.shape, e.decl.init, seed, model.device))
    model.bind()


def write_random_model(config: ModelConfig, seed: int, folder: str | Path, dtype: torch.dtype = torch.bfloat16,
                       device="cpu") -> Path:
    """Writes ``config.json`` and ``model.safetensors`` with random weights stored in ``dtype``.  The
    numbers are drawn on ``device`` (a CUDA device draws a model of billions of weights in seconds; its
    generator gives other numbers than the CPU's for the same seed)."""
    from ..engine.model import DecoderModel

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    raw = config.to_dict()
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    import json

    with open(folder / "config.json", "w") as fh:
        json.dump(raw, fh, indent=2)
    model = DecoderModel(architecture_named(config.architecture).build(config))
    expected = model.expected_tensors()
    plan = [(e.name, dtype, tuple(e.decl.shape)) for e in expected]
    stream = ((e.name, random_tensor(e.name, e.decl.shape, e.decl.init, seed, device).to(dtype).cpu())
              for e in expected)
    write_safetensors(folder / "model.safetensors", stream, plan, metadata={"format": "pt", "seed": str(seed)})
    return folder
