"""RMSNorm: x * (1/sqrt(mean(x^2) + eps)) * w, eps inside the root, plain weight,
32-bit arithmetic (crates/cuda/kernels/dense_kernels.cu:59-88; the residual-fused
form :257-296)."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import Norm, register_part


class RMSNorm(Norm):
    adds_partial_sums = True            # delta may be a stack [S, rows, width] of partial sums

    def __init__(self, width: int, eps: float):
        self.width, self.eps = int(width), float(eps)
        self.weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.width,), init="norm")}

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, ctx, x, out=None, delta=None, row_idx=None):
        rows = x.shape[0] if row_idx is None else row_idx.numel()
        if out is None:
            out = torch.empty((rows, self.width), dtype=ctx.dtype, device=x.device)
        ops.add_rmsnorm(x, delta, self.weight, out, self.eps, row_idx)
        return out


register_part("norm", "rmsnorm", RMSNorm)
