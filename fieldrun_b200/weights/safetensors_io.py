"""Reading and writing safetensors files, and a model folder's tensor index.

The format: 8 bytes little-endian header length, a JSON header mapping each
tensor name to ``dtype``, ``shape`` and ``data_offsets`` within the data section,
then the data.  A folder holds one ``model.safetensors`` or several shards named
by ``model.safetensors.index.json``'s ``weight_map`` -- the two layouts the
reference's converter opens (src/convert.rs:44-63).  Files are memory-mapped and
a tensor is read only when it is asked for.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Callable, Iterable, Sequence

import numpy as np
import torch

# safetensors dtype tag -> (torch dtype, numpy dtype used to view the bytes)
_DTYPES = {
    "F32": (torch.float32, np.dtype("<f4")),
    "F16": (torch.float16, np.dtype("<f2")),
    "BF16": (torch.bfloat16, np.dtype("<u2")),
    "F64": (torch.float64, np.dtype("<f8")),
    "I32": (torch.int32, np.dtype("<i4")),
    "I64": (torch.int64, np.dtype("<i8")),
    "U8": (torch.uint8, np.dtype("u1")),
}
_TAG_OF = {v[0]: k for k, v in _DTYPES.items()}


class WeightFileError(ValueError):
    """A safetensors file or a model folder cannot be read."""


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype_tag: str
    shape: tuple[int, ...]
    file: str
    begin: int          # absolute byte offset in the file
    end: int

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype_tag][0]


def read_header(path: str) -> list[TensorEntry]:
    size = os.path.getsize(path)
    with open(path, "rb") as handle:
        head = handle.read(8)
        if len(head) != 8:
            raise WeightFileError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or 8 + n > size:
            raise WeightFileError(f"{path}: header length {n} does not fit the file of {size} bytes")
        try:
            header = json.loads(handle.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as err:
            raise WeightFileError(f"{path}: header is not valid JSON ({err})") from None
    base = 8 + n
    entries = []
    for name, info in header.items():
        if name == "__metadata__":
            continue
        tag = info.get("dtype")
        if tag not in _DTYPES:
            raise WeightFileError(f"{path}: tensor {name!r} has unsupported dtype {tag!r}")
        shape = tuple(int(s) for s in info["shape"])
        begin, end = (int(o) for o in info["data_offsets"])
        want = int(np.prod(shape, dtype=np.int64)) * _DTYPES[tag][1].itemsize
        if end - begin != want or base + end > size:
            raise WeightFileError(
                f"{path}: tensor {name!r} claims bytes [{begin}, {end}) for shape {list(shape)} {tag}, "
                f"which needs {want} bytes in a data section of {size - base}")
        entries.append(TensorEntry(name, tag, shape, path, base + begin, base + end))
    return entries


class ModelFolder:
    """Index of every tensor of a model folder; tensors are read on demand."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index_path = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        files: list[str]
        if os.path.isfile(index_path):
            with open(index_path, "r", encoding="utf-8") as handle:
                weight_map = json.load(handle).get("weight_map", {})
            files = sorted({os.path.join(model_dir, f) for f in weight_map.values()})
            absent = [f for f in files if not os.path.isfile(f)]
            if absent:
                raise WeightFileError(f"{model_dir}: shard files named by the index are missing: {absent}")
        elif os.path.isfile(single):
            files = [single]
        else:
            raise WeightFileError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json found")
        self.entries: dict[str, TensorEntry] = {}
        for path in files:
            for entry in read_header(path):
                if entry.name in self.entries:
                    raise WeightFileError(f"{model_dir}: tensor {entry.name!r} appears in two files")
                self.entries[entry.name] = entry
        self._maps: dict[str, mmap.mmap] = {}

    def _map(self, path: str) -> mmap.mmap:
        if path not in self._maps:
            with open(path, "rb") as handle:
                self._maps[path] = mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_READ)
        return self._maps[path]

    def names(self) -> list[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """The tensor as a CPU tensor in its stored dtype (a copy; the map may be closed afterwards)."""
        entry = self.entries[name]
        torch_dtype, np_dtype = _DTYPES[entry.dtype_tag]
        count = int(np.prod(entry.shape, dtype=np.int64))
        flat = np.frombuffer(self._map(entry.file), dtype=np_dtype, count=count, offset=entry.begin)
        out = torch.from_numpy(flat.copy())
        if entry.dtype_tag == "BF16":
            out = out.view(torch.bfloat16)
        return out.reshape(entry.shape)

    def close(self) -> None:
        for m in self._maps.values():
            m.close()
        self._maps.clear()


@dataclass(frozen=True)
class TensorToWrite:
    name: str
    shape: tuple[int, ...]
    dtype: torch.dtype
    make: Callable[[], torch.Tensor]


def write_safetensors(path: str, tensors: Sequence[TensorToWrite] | Iterable[tuple[str, torch.Tensor]]) -> None:
    """Write one safetensors file.  Tensors are produced one at a time so that
    a large model never sits in memory whole."""
    items: list[TensorToWrite] = []
    for item in tensors:
        if isinstance(item, TensorToWrite):
            items.append(item)
        else:
            name, value = item
            items.append(TensorToWrite(name, tuple(value.shape), value.dtype, (lambda v=value: v)))
    header: dict[str, object] = {}
    offset = 0
    for item in items:
        if item.dtype not in _TAG_OF:
            raise WeightFileError(f"tensor {item.name!r}: dtype {item.dtype} cannot be written")
        tag = _TAG_OF[item.dtype]
        nbytes = int(np.prod(item.shape, dtype=np.int64)) * _DTYPES[tag][1].itemsize
        header[item.name] = {"dtype": tag, "shape": list(item.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for item in items:
            value = item.make().detach().to("cpu").contiguous()
            if tuple(value.shape) != item.shape or value.dtype != item.dtype:
                raise WeightFileError(
                    f"tensor {item.name!r}: produced {list(value.shape)} {value.dtype}, "
                    f"declared {list(item.shape)} {item.dtype}")
            if value.dtype == torch.bfloat16:
                value = value.view(torch.uint16) if hasattr(torch, "uint16") else value.view(torch.int16)
            handle.write(value.numpy().tobytes())
