"""Helpers shared by the GPU tests: model folders in temporary places, tolerances."""

from __future__ import annotations

import torch

import plain_model
from dryft_flash_infer_b200 import Qwen3Config
from dryft_flash_infer_b200.weights import write_safetensors

#: float32 logits may differ from the plain implementation by summation order only
F32_ATOL = 2e-4
#: bfloat16: 8 significant bits per rounding, a few dozen roundings on the way to a logit
BF16_REL = 0.03


def write_model(folder, cfg: dict, weights: dict, store: torch.dtype = torch.float32):
    Qwen3Config.from_dict(cfg).save(folder)
    write_safetensors(folder / "model.safetensors", ((k, v.to(store)) for k, v in weights.items()))
    return folder


def tolerance(dtype: str, reference: torch.Tensor) -> float:
    if dtype == "float32":
        return F32_ATOL
    return BF16_REL * max(1.0, float(reference.abs().max()))


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = ""):
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: not finite"
    err = float((got - want).abs().max())
    tol = tolerance(dtype, want)
    assert err <= tol, f"{what}: max error {err:.3e} > {tol:.3e} ({dtype})"


def bf16_weights(weights: dict) -> dict:
    """The weights as a bfloat16 engine holds them (matrices rounded, vectors kept), in float32:
    what the plain implementation is given when it is compared with the bfloat16 engine."""
    return {k: (v if v.dim() == 1 else v.to(torch.bfloat16).float()) for k, v in weights.items()}


def prompts_for(cfg: dict, lengths, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]


CONFIGS = {"A": plain_model.TINY_A, "B": plain_model.TINY_B}
