"""SwiGLU feed-forward: down( silu(x Wg^T) * (x Wu^T) ), no bias
(crates/cuda/src/engine.rs:4288-4314; crates/cuda/kernels/dense_kernels.cu:236-248).
Gate and up rows are concatenated once at load into one `[2F, h]` matrix so that one
product serves both (the reference runs two); in bfloat16 that product keeps two
accumulators and applies the activation in its epilogue."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import FeedForward, RowScaled, register_part
from .linear import matmul, matmul_into_residual, takes_row_scaled


class SwiGLU(FeedForward):
    def __init__(self, hidden: int, intermediate: int):
        self.hidden, self.inter = int(hidden), int(intermediate)
        self.w_gate_up = None
        self.w_down = None

    def param_specs(self):
        return {"gate_proj.weight": ParamSpec((self.inter, self.hidden)),
                "up_proj.weight": ParamSpec((self.inter, self.hidden)),
                "down_proj.weight": ParamSpec((self.hidden, self.inter))}

    def bind(self, tensors):
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"]

    @property
    def takes_row_scaled(self) -> bool:
        """The first product (gate and up) can apply the factor of rows that the norm left without it."""
        return takes_row_scaled(self.w_gate_up)

    def forward(self, ctx, xn, residual):
        act = torch.empty((xn.shape[0], self.inter), dtype=xn.dtype, device=xn.device)
        if isinstance(xn, RowScaled):
            if not ops.gemm_bf16_swiglu(xn.rows, self.w_gate_up, act, row_scale=xn.scale()):
                raise ValueError("swiglu: rows without their factor need the tensor-core product")
            return matmul_into_residual(ctx, act, self.w_down, residual)
        fused = xn.dtype == torch.bfloat16 and self.w_gate_up.dtype == torch.bfloat16 and \
            ops.gemm_bf16_swiglu(xn, self.w_gate_up, act)          # activation in the product's epilogue
        if not fused:
            gu = matmul(ctx, xn, self.w_gate_up)
            ops.swiglu(gu, act)
        return matmul_into_residual(ctx, act, self.w_down, residual)


register_part("ffn", "swiglu", SwiGLU)
