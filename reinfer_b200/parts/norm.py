"""RMSNorm: x * (1/sqrt(mean(x^2) + eps)) * w, eps inside the root, plain weight,
32-bit arithmetic (crates/cuda/kernels/dense_kernels.cu:59-88; the residual-fused
form :257-296)."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import Norm, RowScaled, register_part


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

    def forward(self, ctx, x, out=None, delta=None, row_idx=None, scaled_ok=False):
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
