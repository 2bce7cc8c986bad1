"""Safetensors files read by tensor name, and written.

The format is an 8-byte little-endian header length, a JSON header mapping each
tensor name to {dtype, shape, data_offsets}, then the raw little-endian data. The
reader maps each file and validates the header as the reference's does
(src/io/safetensors.cpp:20-60): every failure names the file and the tensor. A model
folder is its `model.safetensors.index.json` shard set, or every `*.safetensors` in
name order, and a name may appear in one file only (src/io/safetensors.cpp:62-104).
"""
from __future__ import annotations

import glob
import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch


class WeightError(RuntimeError):
    """A model's tensors cannot be read or do not fit the configuration."""


# safetensors dtype string -> (torch dtype, bytes per element)
_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class TensorEntry:
    __slots__ = ("name", "dtype", "shape", "begin", "end", "file")

    def __init__(self, name, dtype, shape, begin, end, file):
        self.name, self.dtype, self.shape = name, dtype, tuple(shape)
        self.begin, self.end, self.file = begin, end, file


class SafetensorsFile:
    """One mapped file; tensors come out as views of the mapping (zero copy)."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise WeightError(f"'{path}' is not a safetensors file ({size} bytes)")
        self._f = open(path, "rb")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if header_len == 0 or header_len > size - 8:
            raise WeightError(f"'{path}': header length {header_len} does not fit in a {size}-byte file")
        try:
            header = json.loads(self._map[8:8 + header_len].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightError(f"'{path}': invalid safetensors header: {e}") from None
        if not isinstance(header, dict):
            raise WeightError(f"'{path}': invalid safetensors header: not an object")
        self.data_begin = 8 + header_len
        data_size = size - self.data_begin
        self.metadata: Dict[str, str] = {}
        self.tensors: Dict[str, TensorEntry] = {}
        for name, entry in header.items():
            if name == "__metadata__":
                if isinstance(entry, dict):
                    self.metadata = {k: v for k, v in entry.items() if isinstance(v, str)}
                continue
            try:
                dtype_name, shape, offsets = entry["dtype"], entry["shape"], entry["data_offsets"]
            except (KeyError, TypeError):
                raise WeightError(f"'{path}': tensor '{name}' lacks dtype, shape or data_offsets") from None
            if dtype_name not in _DTYPES:
                raise WeightError(f"'{path}': tensor '{name}' has unsupported dtype {dtype_name}")
            dtype, width = _DTYPES[dtype_name]
            if (not isinstance(offsets, list) or len(offsets) != 2 or offsets[0] > offsets[1]
                    or offsets[1] > data_size):
                raise WeightError(f"'{path}': tensor '{name}' has invalid data_offsets")
            need = width * int(np.prod(shape, dtype=np.int64)) if shape else width
            if offsets[1] - offsets[0] != need:
                raise WeightError(f"'{path}': tensor '{name}' is {offsets[1] - offsets[0]} bytes but "
                                  f"{list(shape)} {dtype_name} needs {need}")
            self.tensors[name] = TensorEntry(name, dtype, shape, offsets[0], offsets[1], self)

    def read(self, entry: TensorEntry) -> torch.Tensor:
        count = int(np.prod(entry.shape, dtype=np.int64)) if entry.shape else 1
        if count == 0:
            return torch.empty(entry.shape, dtype=entry.dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)    # the mapping is read-only; nothing writes to it
            t = torch.frombuffer(self._map, dtype=entry.dtype, count=count,
                                 offset=self.data_begin + entry.begin)
        return t.reshape(entry.shape)


class WeightStore:
    """Every tensor of a model folder, by name."""

    def __init__(self, files: List[SafetensorsFile], where: str):
        self.where = where
        self.files = files
        self.index: Dict[str, TensorEntry] = {}
        for f in files:
            for name, entry in f.tensors.items():
                if name in self.index:
                    raise WeightError(f"tensor '{name}' appears in more than one safetensors file under '{where}'")
                self.index[name] = entry

    @classmethod
    def open_dir(cls, folder: str) -> "WeightStore":
        index_path = os.path.join(folder, "model.safetensors.index.json")
        if os.path.isfile(index_path):
            with open(index_path, "r", encoding="utf-8") as f:
                index = json.load(f)
            shards = sorted(set(index.get("weight_map", {}).values()))
            paths = [os.path.join(folder, s) for s in shards]
        else:
            paths = sorted(glob.glob(os.path.join(folder, "*.safetensors")))
        if not paths:
            raise WeightError(f"no safetensors files in '{folder}'")
        return cls([SafetensorsFile(p) for p in paths], folder)

    def names(self) -> List[str]:
        return list(self.index)

    def __contains__(self, name: str) -> bool:
        return name in self.index

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.index[name].shape

    def dtype(self, name: str) -> torch.dtype:
        return self.index[name].dtype

    def get(self, name: str) -> torch.Tensor:
        """The tensor as stored (a read-only view of the mapped file)."""
        if name not in self.index:
            raise WeightError(f"weight '{name}' not found")
        e = self.index[name]
        return e.file.read(e)


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]],
                      metadata: Optional[Dict[str, str]] = None) -> None:
    """Writes (name, tensor) pairs in the given order; CPU tensors of a dtype above."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    items = []
    offset = 0
    for name, t in tensors:
        if t.dtype not in _NAMES:
            raise WeightError(f"tensor '{name}': dtype {t.dtype} cannot be written")
        t = t.detach().contiguous().cpu()
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        items.append(t)
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)     # data begins on an 8-byte boundary
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for t in items:
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes()
                        if t.numel() * t.element_size() < (1 << 26)
                        else memoryview(t.reshape(-1).view(torch.uint8).numpy()))
    os.replace(tmp, path)
