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
        if out is None:
            return torch.mm(rows, weight.t())
        return torch.mm(rows, weight.t(), out=out)
    result = torch.mm(rows, weight.t(), out_dtype=torch.float32)
    if out is None:
        return result
    out.copy_(result)
    return out
