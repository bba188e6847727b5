"""Reading and writing the safetensors format, by tensor name.

Format: 8 bytes little-endian header length N, N bytes of JSON mapping each name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the
header; ``__metadata__`` is free text), then the raw little-endian data.  A model folder
holds ``model.safetensors`` or shards listed in ``model.safetensors.index.json``.
The file is opened, checked and mapped by a native reader (``csrc/safetensors_reader.cpp``);
tensors are views of the map, so only what is copied to the device is touched.
"""

from __future__ import annotations

import ctypes
import json
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


def _reader():
    """The native reader (``csrc/safetensors_reader.cpp``), compiled at first use."""
    from ..ops import build

    lib = build.load_library("dfi_io", build.IO_SOURCES)
    if not getattr(lib, "_dfi_typed", False):
        lib.dfi_st_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p, ctypes.c_int]
        lib.dfi_st_close.argtypes = [ctypes.c_void_p]
        lib.dfi_st_close.restype = None
        lib.dfi_st_count.argtypes = [ctypes.c_void_p]
        lib.dfi_st_entry.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_char_p),
                                     ctypes.POINTER(ctypes.c_char_p), ctypes.POINTER(ctypes.c_int),
                                     ctypes.POINTER(ctypes.c_longlong), ctypes.c_int,
                                     ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_longlong)]
        lib.dfi_st_metadata.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_longlong)]
        lib.dfi_st_metadata.restype = ctypes.c_void_p
        lib.dfi_st_data.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_longlong)]
        lib.dfi_st_data.restype = ctypes.c_void_p
        lib.dfi_st_read.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int]
        lib._dfi_typed = True
    return lib


class SafetensorsFile:
    """One ``.safetensors`` file, opened, checked and mapped by the native reader: its header, and
    tensors as CPU views of the memory map (``tensor``) or as copies made by several threads
    (``read_into``)."""

    MAX_DIMS = 16
    COPY_THREADS = 8

    def __init__(self, path: str | Path):
        self.path = Path(path)
        self._lib = _reader()
        handle = ctypes.c_void_p()
        err = ctypes.create_string_buffer(1024)
        if self._lib.dfi_st_open(str(self.path).encode(), ctypes.byref(handle), err, len(err)) != 0:
            raise SafetensorsError(err.value.decode(errors="replace"))
        self._handle = handle
        length = ctypes.c_longlong()
        text = self._lib.dfi_st_metadata(self._handle, ctypes.byref(length))
        self.metadata = json.loads(ctypes.string_at(text, length.value)) if text else {}
        size = ctypes.c_longlong()
        self._data = self._lib.dfi_st_data(self._handle, ctypes.byref(size))
        self._data_size = size.value
        self.entries: dict[str, tuple[torch.dtype, tuple[int, ...], int, int]] = {}
        name, dtype = ctypes.c_char_p(), ctypes.c_char_p()
        n_dims, begin, end = ctypes.c_int(), ctypes.c_longlong(), ctypes.c_longlong()
        shape = (ctypes.c_longlong * self.MAX_DIMS)()
        for i in range(self._lib.dfi_st_count(self._handle)):
            if self._lib.dfi_st_entry(self._handle, i, ctypes.byref(name), ctypes.byref(dtype), ctypes.byref(n_dims),
                                      shape, self.MAX_DIMS, ctypes.byref(begin), ctypes.byref(end)) != 0:
                raise SafetensorsError(f"{self.path}: a tensor has more than {self.MAX_DIMS} dimensions")
            label = dtype.value.decode()
            if label not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor '{name.value.decode()}' has unsupported dtype {label}")
            self.entries[name.value.decode()] = (_DTYPES[label], tuple(shape[d] for d in range(n_dims.value)),
                                                 begin.value, end.value)

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            self._lib.dfi_st_close(handle)

    def names(self) -> list[str]:
        return list(self.entries)

    def info(self, name: str) -> tuple[torch.dtype, tuple[int, ...]]:
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU view of the tensor in the read-only map (valid while this object lives)."""
        dtype, shape, begin, end = self.entries[name]
        if begin == end:
            return torch.empty(shape, dtype=dtype)
        window = (ctypes.c_char * (end - begin)).from_address(self._data + begin)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the map is read-only; the view is only ever copied from
            flat = torch.frombuffer(window, dtype=dtype, count=_numel(shape))
        flat._dfi_keep = self            # the map must outlive the view
        return flat.view(shape)

    def read_into(self, name: str, out: torch.Tensor, first_element: int = 0) -> torch.Tensor:
        """Copies ``out.numel()`` elements of the tensor, from ``first_element`` on, into ``out`` (CPU,
        contiguous, the tensor's dtype) with several threads."""
        dtype, shape, begin, end = self.entries[name]
        assert out.device.type == "cpu" and out.is_contiguous() and out.dtype == dtype
        width = out.element_size()
        assert 0 <= first_element and first_element + out.numel() <= _numel(shape)
        if self._lib.dfi_st_read(self._handle, begin + first_element * width, out.numel() * width, out.data_ptr(),
                                 self.COPY_THREADS) != 0:
            raise SafetensorsError(f"{self.path}: tensor '{name}' could not be read")
        return out


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

    def read_into(self, name: str, out: torch.Tensor, first_element: int = 0) -> torch.Tensor:
        return self.where[name].read_into(name, out, first_element)


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
