"""Helpers shared by the GPU tests: model folders in temporary places, tolerances."""

from __future__ import annotations

import torch

import plain_model
from dryft_flash_infer_b200 import Qwen3Config
from dryft_flash_infer_b200.weights import write_safetensors

#: float32 logits may differ from the plain implementation by summation order only
F32_ATOL = 2e-4
#: bfloat16 bounds on the largest logit error, per family of tests: about twice the largest error that the
#: family's tests showed on a B200 (printed at the end of a GPU run, see ``conftest.py``), on logits with a
#: standard deviation of 0.5 to 0.6.  "tiny": the configurations A to D of the tests; "wide": the layers
#: at the widths of Qwen3-4B, whose logits are sums over 2,560 terms.
BF16_ATOL = {"tiny": 0.06, "wide": 0.12}
#: how far below the plain implementation's best logit a token chosen by the bfloat16 engine may lie
BF16_TIE_GAP = 0.05

#: the largest error each family has shown in this run, for the summary at the end
SEEN: dict[tuple[str, str], tuple[float, str]] = {}
#: other measured numbers that bounds rest on, ``name -> text``, printed with the summary
NOTES: dict[str, str] = {}


def write_model(folder, cfg: dict, weights: dict, store: torch.dtype = torch.float32):
    Qwen3Config.from_dict(cfg).save(folder)
    write_safetensors(folder / "model.safetensors", ((k, v.to(store)) for k, v in weights.items()))
    return folder


def tolerance(dtype: str, family: str = "tiny") -> float:
    return F32_ATOL if dtype == "float32" else BF16_ATOL[family]


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "", family: str = "tiny"):
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: not finite"
    err = float((got - want).abs().max())
    if err > SEEN.get((dtype, family), (-1.0, ""))[0]:
        SEEN[(dtype, family)] = (err, what)
    tol = tolerance(dtype, family)
    assert err <= tol, f"{what}: max error {err:.3e} > {tol:.3e} ({dtype})"


def bf16_weights(weights: dict) -> dict:
    """The weights as a bfloat16 engine holds them (matrices rounded, vectors kept), in float32:
    what the plain implementation is given when it is compared with the bfloat16 engine."""
    return {k: (v if v.dim() == 1 else v.to(torch.bfloat16).float()) for k, v in weights.items()}


def prompts_for(cfg: dict, lengths, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]


CONFIGS = {"A": plain_model.TINY_A, "B": plain_model.TINY_B}
