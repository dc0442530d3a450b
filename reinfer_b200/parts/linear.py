"""y = x W^T for a weight kept `[out, in]` as the checkpoint stores it (the
reference transposes at load, crates/cuda/src/engine.rs:6523-6540; here both
operands are K-major, which is what the tensor cores want too).

`matmul` picks the kernel: the tensor-core kernels take bfloat16 x bfloat16; every
other combination (the whole 32-bit path; a weight kept in 32 bits beside 16-bit
activations) runs the plain FMA kernel.  The destination is a new tensor in the
activation dtype, a given tensor, or - with `accumulate=True` - a float32 tensor
that the product is added into (the residual stream).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import RowScaled


def takes_row_scaled(w: Optional[torch.Tensor]) -> bool:
    """Whether products with this weight can apply a row factor in their epilogue (the tensor-core kernel with
    operands that TMA can address): a part whose first product qualifies may accept RowScaled input."""
    return w is not None and w.dtype == torch.bfloat16 and w.is_cuda and \
        w.stride(1) == 1 and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0 and w.shape[1] % 8 == 0


def matmul(ctx, a, w: torch.Tensor, out: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, accumulate: bool = False) -> torch.Tensor:
    """a: a tensor [M, K], or RowScaled rows, whose factor the product's epilogue applies."""
    row_scale = None
    if isinstance(a, RowScaled):
        a, row_scale = a.rows, a.scale()
    M, N = a.shape[0], w.shape[0]
    if out is None:
        if accumulate:
            raise ValueError("matmul: accumulation needs a destination")
        out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
    if accumulate and out.dtype != torch.float32:
        raise ValueError("matmul: accumulation needs a float32 destination")
    if M == 0:
        return out
    if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        ops.gemm_bf16(a, w, out, accumulate, row_scale=row_scale)
    else:
        if row_scale is not None:
            raise ValueError("matmul: rows without their factor need the tensor-core product")
        ops.gemm_ref(a, w, out, accumulate)
    return out


def matmul_into_residual(ctx, a: torch.Tensor, w: torch.Tensor, residual: torch.Tensor) -> Optional[torch.Tensor]:
    """residual += a W^T - now, or by the norm that reads the residual next.

    Where the step lets sums be deferred (ctx.defer_residual: every norm of the model adds stacked
    partial sums) and the product is one of the weight-streaming kind, the product leaves its split
    partial sums [S, T, N] and this returns them: the caller hands them on as its result, and the next
    norm adds them to the residual in a fixed order before it normalises.  Otherwise the product is
    added to the residual here and None is returned.

    Where a block named the norm that reads the residual next (ctx.norm_ahead) and that norm can have its rows made
    by the product itself, the product adds into the residual and this returns those rows (PreparedRows)."""
    norm = getattr(ctx, "norm_ahead", None)
    if norm is not None and a.shape[0] and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        made = norm.prepared_by(ctx, a, w, residual)
        if made is not None:
            return made
    if getattr(ctx, "defer_residual", False):
        parts = ops.gemm_bf16_partials(a, w) if a.shape[0] else None
        if parts is not None:
            return parts
    matmul(ctx, a, w, out=residual, accumulate=True)
    return None
