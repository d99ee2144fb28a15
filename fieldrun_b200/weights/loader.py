"""Weights by tensor name: what the parts need, checked against what a folder holds.

Each part lists its tensors as :class:`TensorNeed` (checkpoint name, shape,
role).  Before any tensor is read the whole list is compared with the folder's
index and one :class:`WeightError` reports every missing tensor, every wrong
shape and every stored type that cannot be read -- the reference stops at the
first missing one (``convert: missing tensor``, src/convert.rs:70,85,95).
Tensors the model has no use for (rotary buffers, heads of other tasks) are
listed in one warning on stderr: the reference fetches by name and never looks
at the rest (src/convert.rs:1231-1257).  ``strict=True`` makes them an error too.

Precision.  A ``matrix`` (an operand of a tensor-core product: projections,
experts, embedding, head) is held in bfloat16 when the model runs in bfloat16,
rounding once if the file stores it wider.  A ``vector`` (norm weights, router
weights and biases: everything used in 32-bit arithmetic) is held in float32
whatever the model's dtype: a tensor stored in 32 bits stays so and a narrower
one is widened, which loses nothing.  A ``table`` of integers becomes int32.  In float32 mode every real tensor is widened to float32, which
is exact for bfloat16 and float16 files (src/convert.rs:74-79 accepts the same
three stored types).
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Callable, Iterable, Mapping, Protocol

import torch

from .safetensors_io import ModelFolder

MATRIX, VECTOR, TABLE = "matrix", "vector", "table"


class WeightError(ValueError):
    """The tensors of a model folder do not fit the model."""

    def __init__(self, where: str, missing: list[str], unexpected: list[str],
                 wrong_shape: list[tuple[str, tuple[int, ...], tuple[int, ...]]],
                 wrong_dtype: list[tuple[str, str]]):
        self.missing, self.unexpected = missing, unexpected
        self.wrong_shape, self.wrong_dtype = wrong_shape, wrong_dtype
        lines = [f"{where}: the tensors do not fit the model"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        for name, want, found in wrong_shape:
            lines.append(f"  wrong shape: {name} expected {list(want)}, found {list(found)}")
        for name, tag in wrong_dtype:
            lines.append(f"  unsupported dtype: {name} is stored as {tag}")
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class TensorNeed:
    name: str                    # name in the checkpoint
    shape: tuple[int, ...]
    role: str = MATRIX           # MATRIX | VECTOR | TABLE
    init: str = "normal"         # random-weights rule: "normal" | "around_one" | "bias"


class TensorSource(Protocol):
    """Where parts fetch their tensors from (a folder, or tensors made in memory)."""

    def fetch(self, need: TensorNeed) -> torch.Tensor: ...


_REAL = {"F32", "F16", "BF16", "F64"}
_INTEGER = {"I32", "I64", "U8"}


def check_needs(where: str, needs: Iterable[TensorNeed], found: Mapping[str, tuple[str, tuple[int, ...]]],
                strict: bool = False) -> list[str]:
    """Raise one WeightError unless ``found`` (name -> (dtype tag, shape)) holds everything ``needs`` lists, in
    the right shapes and readable types.  Returns the names the model has no use for (an error if ``strict``)."""
    wanted: dict[str, TensorNeed] = {}
    for need in needs:
        other = wanted.get(need.name)
        if other is not None and other.shape != need.shape:
            raise ValueError(f"tensor {need.name!r} is needed with two shapes: {other.shape} and {need.shape}")
        wanted[need.name] = need
    missing = [n for n in wanted if n not in found]
    unexpected = [n for n in found if n not in wanted]
    wrong_shape, wrong_dtype = [], []
    for name, need in wanted.items():
        if name not in found:
            continue
        tag, shape = found[name]
        if tuple(shape) != tuple(need.shape):
            wrong_shape.append((name, tuple(need.shape), tuple(shape)))
        allowed = _INTEGER if need.role == TABLE else _REAL
        if tag not in allowed:
            wrong_dtype.append((name, tag))
    if missing or wrong_shape or wrong_dtype or (strict and unexpected):
        raise WeightError(where, missing, unexpected, wrong_shape, wrong_dtype)
    return unexpected


def held_dtype(role: str, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    """The dtype a tensor is held in on the device (see the module's note on precision)."""
    if role == TABLE:
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if role == MATRIX:
        return torch.bfloat16
    return torch.float32


class FolderSource:
    """Tensors of a model folder, validated against the model's needs up front."""

    def __init__(self, model_dir: str, needs: Iterable[TensorNeed], compute_dtype: torch.dtype,
                 device: torch.device | str, strict: bool = False):
        self.folder = ModelFolder(model_dir)
        found = {n: (e.dtype_tag, e.shape) for n, e in self.folder.entries.items()}
        self.unused = check_needs(model_dir, needs, found, strict)
        if self.unused:
            shown = ", ".join(self.unused[:8]) + (f", ... ({len(self.unused)} in all)" if len(self.unused) > 8 else "")
            print(f"{model_dir}: warning: tensors the model has no use for are left unread: {shown}", file=sys.stderr)
        self.compute_dtype = compute_dtype
        self.device = torch.device(device)

    def fetch(self, need: TensorNeed) -> torch.Tensor:
        value = self.folder.tensor(need.name)
        target = held_dtype(need.role, value.dtype, self.compute_dtype)
        return value.to(device=self.device, dtype=target).contiguous()

    def close(self) -> None:
        self.folder.close()


class MemorySource:
    """Tensors made by a function of the need (random weights made on the device)."""

    def __init__(self, make: Callable[[TensorNeed], torch.Tensor], stored_dtype: Callable[[TensorNeed], torch.dtype],
                 compute_dtype: torch.dtype, device: torch.device | str):
        self.make, self.stored_dtype = make, stored_dtype
        self.compute_dtype, self.device = compute_dtype, torch.device(device)

    def fetch(self, need: TensorNeed) -> torch.Tensor:
        value = self.make(need)
        if tuple(value.shape) != tuple(need.shape):
            raise ValueError(f"tensor {need.name!r}: made {list(value.shape)}, needed {list(need.shape)}")
        target = held_dtype(need.role, self.stored_dtype(need), self.compute_dtype)
        return value.to(device=self.device, dtype=target).contiguous()
