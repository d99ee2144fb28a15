"""RMSNorm: x * (1 / sqrt(mean(x^2) + eps)) * w per row, the weight used as it is
(src/minimax.rs:56-66).  The kernel also performs the residual sum that precedes
the norm, in float32, so the update of the stream and the norm read it once."""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import VECTOR, TensorNeed, TensorSource
from .base import Norm, WeightedRows, as_tensor, register_part


class RMSNorm(Norm):
    replayable = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.width = int(spec.args["width"])
        self.eps = float(spec.args["eps"])
        self.weight: Optional[torch.Tensor] = None

    def tensor_needs(self):
        return [TensorNeed(self.name_of("weight"), (self.width,), VECTOR, "around_one")]

    def load(self, source: TensorSource) -> None:
        self.weight = source.fetch(self.tensor_needs()[0])

    accepts_deferred = True

    def forward(self, ctx, x, *, delta=None, rows=None, want32=False, write_back=True):
        experts = None
        if isinstance(delta, WeightedRows) and delta.top_k <= ops.NORM_MAX_SUMMED_ROWS:
            experts, delta = (delta.rows, delta.weights, delta.row_map), None      # the kernel sums them as it reads x
        else:
            delta = as_tensor(ctx, delta)
        count = rows.numel() if rows is not None else x.shape[0]
        out = ctx.buffer(f"norm.out.{self.width}", (count, self.width), self.dtype)
        out32 = None
        if want32:
            out32 = out if self.dtype == torch.float32 else ctx.buffer(f"norm.out32.{self.width}", (count, self.width),
                                                                       torch.float32)
        ops.rmsnorm(x, self.weight, self.eps, out, delta=delta, rows=rows, out32=None if out32 is out else out32,
                    write_back=write_back and (delta is not None or experts is not None), experts=experts)
        return out, out32


register_part("norm", "rmsnorm", RMSNorm, replace=True)
