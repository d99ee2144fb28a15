"""Plain dense matrix products through the library (cuBLAS via torch.mm).

The reference's dense products (``Bundle::mm``, src/bundle.rs:644-683) are a
library call as well: ndarray's ``dot`` over matrixmultiply or cblas.  Weights
stay in the checkpoint's ``(out, in)`` layout; the product is ``rows @ W^T``
with float32 accumulation and a float32 result.  In float32 mode the reduced
precision matrix modes (TF32, bf16 reductions) are switched off and that is
checked at every call.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops

_ONE_TILE: dict[tuple[str, int], tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]] = {}
STREAM_ROWS = 8           # up to this many rows a dense product is a stream over the weight (experts_stream.cu); beyond, each
                          # item's rows of x are as many bytes as its weights and the library's product is faster (measured at
                          # 12 to 32 rows on a B200: 14 to 25 us against 11 for MiniMax-M2's projections)
STREAM_FEATURES = 65536   # beyond this many output features the library product is at the memory roofline anyway


def _one_tile(device: torch.device, rows: int):
    key = (str(device), rows)
    if key not in _ONE_TILE:
        zero = torch.zeros(1, dtype=torch.int32, device=device)
        _ONE_TILE[key] = (zero, zero.clone(), torch.ones(1, dtype=torch.int32, device=device),
                          torch.tensor([0, rows], dtype=torch.int32, device=device))
    return _ONE_TILE[key]


def require_true_float32() -> None:
    """Switch off every reduced-precision mode of float32 matrix products."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    if hasattr(torch.backends.cuda.matmul, "allow_bf16_reduced_precision_reduction"):
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    if hasattr(torch.backends.cuda.matmul, "allow_fp16_reduced_precision_reduction"):
        torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False


def linear(rows: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """rows [T, in] @ weight[out, in]^T -> float32 [T, out]."""
    if not rows.is_cuda:
        raise RuntimeError("fieldrun_b200 runs on a CUDA device only; a CPU tensor reached a matrix product")
    if rows.dtype != weight.dtype:
        raise RuntimeError(f"matrix product of {rows.dtype} rows with a {weight.dtype} weight")
    if rows.dtype == torch.float32:
        if torch.backends.cuda.matmul.allow_tf32 or torch.get_float32_matmul_precision() != "highest":
            raise RuntimeError("a float32 matrix product was asked for while TF32 is allowed")
        with ops.timed(f"library_mm_f32[{weight.shape[0]}x{weight.shape[1]}]"):
            if out is None:
                return torch.mm(rows, weight.t())
            return torch.mm(rows, weight.t(), out=out)
    count, inner = rows.shape
    features = weight.shape[0]
    if count <= STREAM_ROWS and inner % 32 == 0 and features % 16 == 0 and features <= STREAM_FEATURES \
            and rows.is_contiguous() and weight.is_contiguous():
        # few rows: the weight is the traffic; stream it once through the kernel that streams expert weights,
        # the dense layer being a single expert whose rows are all the rows
        tile_rows = 8 if count <= 8 else 16 if count <= 16 else 32
        tile_expert, tile_row0, num_tiles, offsets = _one_tile(rows.device, count)
        result = out if out is not None else torch.empty((count, features), dtype=torch.float32, device=rows.device)
        if ops.weight_stream_takes(features, inner, paired=False):
            # the lists of this one tile never change, so the weights may be on their way before the rows are ready
            ops.weight_stream(weight.view(1, features, inner), rows, None, tile_expert, tile_row0, num_tiles, offsets, 1,
                              tile_rows, result, paired=False, lists_final=True)
        else:
            ops.expert_gemm_mma(weight.view(1, features, inner), rows, None, tile_expert, tile_row0, num_tiles, offsets, 1,
                                tile_rows, result, paired=False, **ops.stream_shape(1, features, inner, tile_rows))
        return result
    with ops.timed(f"library_mm[{features}x{inner}]"):
        result = torch.mm(rows, weight.t(), out_dtype=torch.float32)
    if out is None:
        return result
    out.copy_(result)
    return out
