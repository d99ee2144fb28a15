"""Rotary position encoding as tables of cos and sin over positions.

The angle of pair j at position p is p * theta^(-2j / rotary_dim), j < rotary_dim/2
(src/minimax.rs:50,76 with rotary_dim = head_dim; the partial form with
rotary_dim < head_dim is src/qwen35moe.rs:78-81,121-138).  The reference forms
the angle and its cos/sin in float32 for every element; here the table is
computed once on the host in float64 and rounded to float32, which is at least
as close to the exact angle.  ``pairing`` "half" rotates (j, j + rotary_dim/2) as
the reference does; "interleaved" rotates (2j, 2j+1).
"""
from __future__ import annotations

import torch

from .base import Position, register_part


class Rotary(Position):
    def __init__(self, args):
        self.rotary_dim = int(args["rotary_dim"])
        self.theta = float(args["theta"])
        pairing = args.get("pairing", "half")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing {pairing!r} is neither 'half' nor 'interleaved'")
        if self.rotary_dim % 2:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even")
        self.interleaved = pairing == "interleaved"
        self.position_scale = float(args.get("position_scale", 1.0))

    def tables(self, num_positions: int, device):
        half = self.rotary_dim // 2
        if half == 0:
            return None, None
        j = torch.arange(half, dtype=torch.float64)
        inv = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64), 2.0 * j / self.rotary_dim)
        pos = torch.arange(num_positions, dtype=torch.float64) * self.position_scale
        angle = pos[:, None] * inv[None, :]
        return (torch.cos(angle).to(torch.float32).to(device).contiguous(),
                torch.sin(angle).to(torch.float32).to(device).contiguous())


register_part("position", "rotary", Rotary, replace=True)
