"""Rotary position encoding, half-split pairing (p, p + rot/2):
angle = pos * theta^(-2p/rot); x'[p] = x[p] cos - x[p+rot/2] sin;
x'[p+rot/2] = x[p] sin + x[p+rot/2] cos   (crates/kernels/src/refs.rs:25-37,
crates/cuda/kernels/dense_kernels.cu:127-170).  The reference evaluates powf per
element on the device; here theta^(-2p/rot) is tabulated once in double precision
and rounded to float32, the angle and its sine and cosine are float32 on the device.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import PositionEncoding, register_part


class RotaryEncoding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, rotary_dim: int = 0):
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim) or self.head_dim
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary width {self.rotary_dim} of head_dim {self.head_dim}")
        self.inv_freq = None

    def table(self) -> torch.Tensor:
        p = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        return (torch.tensor(self.theta, dtype=torch.float64) ** (-(2.0 * p) / self.rotary_dim)).to(torch.float32)

    def prepare(self, device) -> None:
        self.inv_freq = self.table().to(device)

    def fused_rotary(self):
        return self.inv_freq, self.rotary_dim

    def table_key(self):
        return ("rope", self.theta, self.rotary_dim)

    def apply(self, ctx, q, k, positions) -> None:
        """The unfused form, for a mixer that does not take `fused_rotary()`: q [T, QH, d] and k [T, KH, d]
        are rotated in place (through the same kernel, with the head norm and the cache switched off)."""
        for x in (q, k):
            T, heads, d = x.shape
            out = torch.empty_like(x)
            ops.qknorm_rope_append(x.reshape(T, heads * d), None, None, self.inv_freq, positions, None, out, None,
                                   heads, 0, d, self.rotary_dim, 1, 0.0)
            x.copy_(out)


register_part("position", "rope", RotaryEncoding)
register_part("position", "none", lambda **kw: None)
