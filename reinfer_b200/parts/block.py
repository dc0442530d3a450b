"""Arrangements of a layer's four parts.  'prenorm':
    x += mixer(norm1(x));  x += ffn(norm2(x))       (crates/cuda/src/engine.rs:4071-4333)
Mixer and feed-forward add into the residual stream themselves (their last product
accumulates into it), so no separate residual kernel runs."""
from __future__ import annotations

from .base import register_part


class PreNormBlock:
    def __init__(self, mixer_norm, mixer, ffn_norm, ffn):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def forward(self, ctx, x, cache) -> None:
        xn = self.mixer_norm.forward(ctx, x)
        self.mixer.forward(ctx, xn, x, cache)
        xn = self.ffn_norm.forward(ctx, x)
        self.ffn.forward(ctx, xn, x)


register_part("block", "prenorm", PreNormBlock)
