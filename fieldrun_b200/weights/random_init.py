"""Random weights from a configuration and a seed.

The reference has no random weights of its own; its gate builds a tiny model
in another framework, redraws the norm weights as N(0, 0.1) + mean and the
routing bias as N(0, 0.2) so that neither is invisible (scripts/gemma3_ref.py:206-247).
The same idea here without that framework: each tensor is drawn from a generator
keyed by the seed and the tensor's name, so a tensor's values do not depend on
the order of drawing or on which other tensors exist.
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


@dataclass(frozen=True)
class RandomInit:
    seed: int = 0
    matrix_std: float = 0.02          # projections, experts, embedding, head: N(0, matrix_std)
    norm_std: float = 0.1             # norm weights: 1 + N(0, norm_std)
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
        gen = torch.Generator(device=device)
        gen.manual_seed((self.seed * 1_000_003 + zlib.crc32(need.name.encode("utf-8"))) % (2 ** 63))
        shape = tuple(need.shape)
        if need.role == TABLE:
            raise ValueError(f"tensor {need.name!r}: integer tables have no random rule")
        if need.init == "around_one":
            value = 1.0 + self.norm_std * torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        elif need.init == "bias":
            if self.bias_std == 0.0:
                value = torch.zeros(shape, device=device, dtype=torch.float32)
            else:
                value = self.bias_std * torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        elif need.init == "normal":
            value = self.matrix_std * torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
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
