"""Reading and writing the safetensors format, by tensor name.

Format: 8 bytes little-endian header length N, N bytes of JSON mapping each name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the
header; ``__metadata__`` is free text), then the raw little-endian data.  A model folder
holds ``model.safetensors`` or shards listed in ``model.safetensors.index.json``.
Tensors are read through a memory map, so only what is copied to the device is touched.
"""

from __future__ import annotations

import json
import mmap
import struct
import warnings
from pathlib import Path
from typing import Iterable

import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


class SafetensorsFile:
    """One ``.safetensors`` file: its header, and tensors as CPU views of the memory map."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        size = self.path.stat().st_size
        with open(self.path, "rb") as fh:
            head = fh.read(8)
            if len(head) < 8:
                raise SafetensorsError(f"{self.path}: truncated (no header length)")
            (n,) = struct.unpack("<Q", head)
            if n > size - 8:
                raise SafetensorsError(f"{self.path}: truncated (header of {n} bytes, file of {size})")
            try:
                header = json.loads(fh.read(n))
            except (json.JSONDecodeError, UnicodeDecodeError) as exc:
                raise SafetensorsError(f"{self.path}: header is not valid JSON ({exc})") from exc
        self.data_start = 8 + n
        self.metadata = header.pop("__metadata__", {})
        self.entries: dict[str, tuple[torch.dtype, tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            if info["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor '{name}' has unsupported dtype {info['dtype']}")
            dtype = _DTYPES[info["dtype"]]
            shape = tuple(int(s) for s in info["shape"])
            begin, end = info["data_offsets"]
            want = _numel(shape) * torch.empty((), dtype=dtype).element_size()
            if end - begin != want:
                raise SafetensorsError(f"{self.path}: tensor '{name}' spans {end - begin} bytes, shape needs {want}")
            if self.data_start + end > size:
                raise SafetensorsError(f"{self.path}: truncated (tensor '{name}' ends past the file)")
            self.entries[name] = (dtype, shape, begin, end)
        self._map = None

    def names(self) -> list[str]:
        return list(self.entries)

    def info(self, name: str) -> tuple[torch.dtype, tuple[int, ...]]:
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, begin, end = self.entries[name]
        if begin == end:
            return torch.empty(shape, dtype=dtype)
        if self._map is None:
            with open(self.path, "rb") as fh:
                self._map = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the map is read-only; the view is only ever copied from
            flat = torch.frombuffer(self._map, dtype=dtype, count=_numel(shape), offset=self.data_start + begin)
        return flat.view(shape)


class ModelFiles:
    """All tensors of a model folder, whichever shard holds them."""

    def __init__(self, folder: str | Path):
        folder = Path(folder)
        index = folder / "model.safetensors.index.json"
        single = folder / "model.safetensors"
        self.files: list[SafetensorsFile] = []
        self.where: dict[str, SafetensorsFile] = {}
        if index.is_file():
            with open(index) as fh:
                shard_names = sorted(set(json.load(fh)["weight_map"].values()))
            paths = [folder / s for s in shard_names]
        elif single.is_file():
            paths = [single]
        else:
            raise SafetensorsError(f"no model.safetensors (or model.safetensors.index.json) in {folder}")
        for path in paths:
            if not path.is_file():
                raise SafetensorsError(f"shard {path} named by the index is missing")
            shard = SafetensorsFile(path)
            self.files.append(shard)
            for name in shard.names():
                if name in self.where:
                    raise SafetensorsError(f"tensor '{name}' is in both {self.where[name].path.name} and {path.name}")
                self.where[name] = shard

    def names(self) -> list[str]:
        return list(self.where)

    def info(self, name: str):
        return self.where[name].info(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self.where[name].tensor(name)


def write_safetensors(path: str | Path, tensors: Iterable[tuple[str, torch.Tensor]], plan=None,
                      metadata: dict[str, str] | None = None) -> None:
    """Writes ``tensors`` (name, tensor) in order.

    With ``plan`` (a list of ``(name, dtype, shape)`` for the same names in the same
    order) the header is written first and the tensors are streamed one by one, so a
    large model never sits in host memory whole; without it ``tensors`` is held as a list.
    """
    if plan is None:
        tensors = [(n, t.detach().contiguous().cpu()) for n, t in tensors]
        plan = [(n, t.dtype, tuple(t.shape)) for n, t in tensors]
    header, offset = {}, 0
    if metadata:
        header["__metadata__"] = metadata
    for name, dtype, shape in plan:
        if dtype not in _NAMES:
            raise SafetensorsError(f"cannot write dtype {dtype}")
        nbytes = _numel(shape) * torch.empty((), dtype=dtype).element_size()
        header[name] = {"dtype": _NAMES[dtype], "shape": list(shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for (name, tensor), (want_name, dtype, shape) in zip(tensors, plan):
            if name != want_name or tensor.dtype != dtype or tuple(tensor.shape) != tuple(shape):
                raise SafetensorsError(f"tensor '{name}' does not match the write plan entry '{want_name}'")
            flat = tensor.detach().contiguous().cpu().view(-1)
            if flat.numel():
                fh.write(flat.view(torch.uint8).numpy().tobytes())
