"""Random weights from a configuration and a seed.

The reference has no random weights of its own; its gate builds a tiny model
in another framework, redraws the norm weights as N(0, 0.1) + mean and the
routing bias as N(0, 0.2) so that neither is invisible (scripts/gemma3_ref.py:206-247).
The same idea here without that framework.  Every element is a function of
(seed, tensor name, element index) alone: a counter-based hash gives 128 bits per
element, their eight 16-bit fields are summed (integer arithmetic) and the centred
sum is scaled by one float32 constant.  Nothing in that depends on a device's
math library or on the order of drawing, so a CPU and a GPU make the same bits
for the same seed, a large model can be made on the device without ever existing
on the host, and a slice of it can be re-made anywhere.  The sum of eight
uniform fields is close to a normal variable for the purpose (unit variance,
bounded at 4.9 sigma, excess kurtosis -0.15).
"""
from __future__ import annotations

import json
import os
import zlib
from dataclasses import dataclass
from typing import Iterable

import torch

from .loader import MATRIX, TABLE, VECTOR, TensorNeed
from .safetensors_io import TensorToWrite, write_safetensors


_MASK = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15
_MUL_A = 0xBF58476D1CE4E5B9
_MUL_B = 0x94D049BB133111EB
_CHUNK = 1 << 24                  # elements drawn at a time (bounds the temporaries at a few hundred MB)
# the sum of eight independent 16-bit fields has variance 8 (2^32 - 1) / 12; twice the centred sum is an integer
_UNIT = 1.0 / (2.0 * (8.0 * (2.0 ** 32 - 1.0) / 12.0) ** 0.5)


def _signed(value: int) -> int:
    """The int64 with the bits of an unsigned 64-bit value."""
    value &= _MASK
    return value - (1 << 64) if value >> 63 else value


def _mix_int(z: int) -> int:
    z = (z + _GOLDEN) & _MASK
    z = ((z ^ (z >> 30)) * _MUL_A) & _MASK
    z = ((z ^ (z >> 27)) * _MUL_B) & _MASK
    return z ^ (z >> 31)


def tensor_key(seed: int, name: str) -> int:
    """64 bits that stand for (seed, tensor name)."""
    return _mix_int(_mix_int(seed & _MASK) ^ zlib.crc32(name.encode("utf-8")))


def _shift_right(z: torch.Tensor, bits: int) -> torch.Tensor:
    """Logical shift of the 64-bit patterns held in an int64 tensor."""
    return (z >> bits) & ((1 << (64 - bits)) - 1)


def _mix(z: torch.Tensor) -> torch.Tensor:
    """The SplitMix64 finaliser on int64 tensors (products wrap around, as unsigned ones do)."""
    z = z + _signed(_GOLDEN)
    z = (z ^ _shift_right(z, 30)) * _signed(_MUL_A)
    z = (z ^ _shift_right(z, 27)) * _signed(_MUL_B)
    return z ^ _shift_right(z, 31)


def _fields(z: torch.Tensor) -> torch.Tensor:
    """The sum of the four 16-bit fields of each 64-bit pattern."""
    return (z & 0xFFFF) + (_shift_right(z, 16) & 0xFFFF) + (_shift_right(z, 32) & 0xFFFF) + _shift_right(z, 48)


def unit_normal(key: int, shape, device, scale: float = 1.0, first: int = 0) -> torch.Tensor:
    """float32 ``scale * z`` with z close to N(0, 1); element i (counted from ``first`` in the flattened
    tensor) depends on ``key`` and i alone, and the bits are the same on every device."""
    count = 1
    for n in shape:
        count *= int(n)
    out = torch.empty(count, dtype=torch.float32, device=device)
    factor = float(torch.tensor(_UNIT * float(scale), dtype=torch.float64).to(torch.float32))
    for begin in range(0, count, _CHUNK):
        end = min(begin + _CHUNK, count)
        index = torch.arange(first + begin, first + end, dtype=torch.int64, device=device)
        a = _mix(index * _signed(_GOLDEN) + _signed(key))
        b = _mix(a)
        total = _fields(a) + _fields(b)                      # 0 .. 8 * 65535
        out[begin:end] = (2 * total - 8 * 65535).to(torch.float32) * factor
    return out.view(*shape) if shape else out.view(())


@dataclass(frozen=True)
class RandomInit:
    seed: int = 0
    matrix_std: float = 0.02          # projections, experts, embedding, head: N(0, matrix_std)
    norm_std: float = 0.1             # norm weights: norm_mean + N(0, norm_std)
    norm_mean: float = 1.0
    bias_std: float = 0.0             # routing bias: N(0, bias_std), zeros when 0
    stored_dtype: torch.dtype = torch.bfloat16
    vectors_in_float32: bool = True   # norm/router tensors are stored in 32-bit

    def stored(self, need: TensorNeed) -> torch.dtype:
        if need.role == TABLE:
            return torch.int32
        if need.role == VECTOR and self.vectors_in_float32:
            return torch.float32
        return self.stored_dtype

    def draw(self, need: TensorNeed, device: torch.device | str = "cpu") -> torch.Tensor:
        device = torch.device(device)
        shape = tuple(need.shape)
        if need.role == TABLE:
            raise ValueError(f"tensor {need.name!r}: integer tables have no random rule")
        key = tensor_key(self.seed, need.name)
        if need.init == "around_one":
            value = unit_normal(key, shape, device, self.norm_std).add_(self.norm_mean)
        elif need.init == "bias":
            if self.bias_std == 0.0:
                value = torch.zeros(shape, device=device, dtype=torch.float32)
            else:
                value = unit_normal(key, shape, device, self.bias_std)
        elif need.init == "normal":
            value = unit_normal(key, shape, device, self.matrix_std)
        else:
            raise ValueError(f"tensor {need.name!r}: unknown random rule {need.init!r}")
        return value.to(self.stored(need))


def write_model_folder(folder: str, config_json: dict, needs: Iterable[TensorNeed], init: RandomInit) -> None:
    """Write ``config.json`` and ``model.safetensors`` of a randomly initialised model."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(config_json, handle, indent=1, sort_keys=True)
    seen: set[str] = set()
    items = []
    for need in needs:
        if need.name in seen:          # a tied tensor is needed twice and written once
            continue
        seen.add(need.name)
        items.append(TensorToWrite(need.name, tuple(need.shape), init.stored(need),
                                   (lambda n=need: init.draw(n, "cpu"))))
    write_safetensors(os.path.join(folder, "model.safetensors"), items)


__all__ = ["RandomInit", "write_model_folder", "MATRIX", "VECTOR", "TABLE"]
