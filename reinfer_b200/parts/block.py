"""Arrangements of a layer's parts.  A block class is constructed with the layer's parts by
role (`Block(parts: dict role -> part)`), says with `roles` which ones it needs, and runs the
layer on the residual stream in `forward(ctx, x, cache)`.  'prenorm':
    x += mixer(mixer_norm(x));  x += ffn(ffn_norm(x))       (crates/cuda/src/engine.rs:4071-4333)
Mixer and feed-forward add into the residual stream themselves (their last product
accumulates into it), so no separate residual kernel runs.  Either may instead return
what is still to be added (a tensor of x's shape, or a stack [S, T, h] of partial sums):
the block hands it to the norm that reads x next, which adds it on the way; what the
feed-forward leaves is the block's own result, for the norm of the next block."""
from __future__ import annotations

from .base import register_part


def need_roles(block_name: str, parts, roles) -> None:
    missing = [r for r in roles if r not in parts]
    if missing:
        raise ValueError(f"block '{block_name}' needs the roles {list(roles)}; the layer lacks {missing} "
                         f"(it has {list(parts)})")


class PreNormBlock:
    roles = ("mixer_norm", "mixer", "ffn_norm", "ffn")
    hands_on_sums = True                # forward takes and returns what is still to be added to x

    def __init__(self, parts):
        need_roles("prenorm", parts, self.roles)
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = (parts[r] for r in self.roles)

    def forward(self, ctx, x, cache, delta=None):
        """Runs the layer on the residual stream x (in place).  delta: what the block before left to be
        added to x first.  Returns what this block leaves to be added (None: nothing)."""
        xn = _norm(self.mixer_norm, self.mixer, ctx, x, delta)
        after = getattr(ctx, "norm_after_block", None)
        ctx.norm_ahead = self.ffn_norm if _prepares(self.ffn_norm, self.ffn) else None
        try:
            delta = self.mixer.forward(ctx, xn, x, cache)
            xn = _norm(self.ffn_norm, self.ffn, ctx, x, delta)
            ctx.norm_ahead = after
            return self.ffn.forward(ctx, xn, x)
        finally:
            ctx.norm_ahead = None

    def entry_norm(self):
        """The norm that reads the residual stream first in this block, if the part before this block may do that
        norm's work in its last product (else None)."""
        return self.mixer_norm if _prepares(self.mixer_norm, self.mixer) else None


def _prepares(norm, reader) -> bool:
    """Whether a product before `norm` may make the norm's rows itself: the norm knows how and hands rows without
    their factor to a reader that takes them."""
    return hasattr(norm, "prepared_by") and getattr(norm, "leaves_row_scale", False) and getattr(reader, "takes_row_scaled", False)


def _norm(norm, reader, ctx, x, delta):
    """The norm before `reader`; rows without their factor only where both sides know of them."""
    if getattr(norm, "leaves_row_scale", False) and getattr(reader, "takes_row_scaled", False):
        return norm.forward(ctx, x, delta=delta, scaled_ok=True)
    return norm.forward(ctx, x, delta=delta)


register_part("block", "prenorm", PreNormBlock)
