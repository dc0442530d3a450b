"""RMSNorm: x * (1/sqrt(mean(x^2) + eps)) * w, eps inside the root, plain weight,
32-bit arithmetic (crates/cuda/kernels/dense_kernels.cu:59-88; the residual-fused
form :257-296)."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import Norm, PreparedRows, RowScaled, register_part


class RMSNorm(Norm):
    adds_partial_sums = True            # delta may be a stack [S, rows, width] of partial sums
    leaves_row_scale = True             # forward(..., scaled_ok=True) may return a RowScaled

    def __init__(self, width: int, eps: float):
        self.width, self.eps = int(width), float(eps)
        self.weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.width,), init="norm")}

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def prepared_by(self, ctx, a, w, residual):
        """residual += a w^T by a product that also makes this norm's rows of the new residual (a decode step's few
        rows, bfloat16): PreparedRows for forward(..., delta=that, scaled_ok=True), or None where that form does not
        apply and nothing was done."""
        if self.weight is None or ctx.dtype != torch.bfloat16 or not ops.DEFER_SUMS or residual.shape[1] != self.width:
            return None
        made = ops.gemm_bf16_residual_norm(a, w, residual, self.weight)
        return None if made is None else PreparedRows(self, made[0], made[1])

    def forward(self, ctx, x, out=None, delta=None, row_idx=None, scaled_ok=False):
        if isinstance(delta, PreparedRows):
            if delta.norm is not self or not scaled_ok or out is not None or row_idx is not None:
                raise ValueError("rmsnorm: rows prepared by a product are for the norm and the reader they were made for")
            return RowScaled(delta.rows, delta.sumsq, self.width, self.eps)
        if scaled_ok and out is None and row_idx is None and ctx.dtype == torch.bfloat16 and ops.DEFER_SUMS and \
                0 < x.shape[0] <= ops.STREAMING_TOKENS and self.width % 4 == 0 and \
                (delta is None or delta.dtype == torch.float32):
            # a decode step's few rows: the division is left to the product that reads them, so that no CTA
            # of this kernel has to wait for a row's whole sum
            y, sumsq = ops.residual_rowscale(x, delta, self.weight)
            return RowScaled(y, sumsq, self.width, self.eps)
        rows = x.shape[0] if row_idx is None else row_idx.numel()
        if out is None:
            out = torch.empty((rows, self.width), dtype=ctx.dtype, device=x.device)
        ops.add_rmsnorm(x, delta, self.weight, out, self.eps, row_idx)
        return out


register_part("norm", "rmsnorm", RMSNorm)
