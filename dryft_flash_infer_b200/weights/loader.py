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


_STAGED_FROM = 4 << 20       # tensors of this many bytes or more go through pinned staging memory
_STAGE_BYTES = 64 << 20


class _Staging:
    """Two pinned buffers used in turn; a buffer is reused only after its copy to the device is done."""

    def __init__(self, device):
        self.device = device
        self.buffers = [torch.empty(_STAGE_BYTES, dtype=torch.uint8).pin_memory() for _ in range(2)]
        self.events = [None, None]
        self.turn = 0

    def next(self, dtype: torch.dtype, count: int) -> torch.Tensor:
        event = self.events[self.turn]
        if event is not None:
            event.synchronize()
        return self.buffers[self.turn].view(dtype)[:count]

    def sent(self) -> None:
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream(self.device))
        self.events[self.turn] = event
        self.turn ^= 1


def load_weights(model, folder: str | Path) -> None:
    """Copies every expected tensor from ``folder`` into ``model``'s allocated buffers."""
    files = ModelFiles(folder)
    expected = model.expected_tensors()
    check_tensors(folder, files, expected, model.spec.ignorable_tensors)
    staging = None
    for e in expected:
        dest = model.destination(e)
        dtype, shape = files.info(e.name)
        n = dest.numel()
        if dest.is_cuda and dest.is_contiguous() and n * torch.empty((), dtype=dtype).element_size() >= _STAGED_FROM:
            # large tensors: the native reader fills pinned memory with several threads, piece by piece,
            # while the piece before is on its way to the device
            staging = staging or _Staging(dest.device)
            flat = dest.view(-1)
            per = _STAGE_BYTES // torch.empty((), dtype=dtype).element_size()
            for at in range(0, n, per):
                host = staging.next(dtype, min(per, n - at))
                files.read_into(e.name, host, at)
                flat[at: at + host.numel()].copy_(host, non_blocking=True)
                staging.sent()
        else:
            dest.copy_(files.tensor(e.name))
    if staging is not None:
        torch.cuda.synchronize(staging.device)
    model.bind()


__all__ = ["WeightError", "SafetensorsError", "check_tensors", "load_weights"]
