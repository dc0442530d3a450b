"""Interfaces of the parts and the registry that maps a kind to a class.

Categories: 'norm', 'position', 'mixer', 'ffn', 'block', 'embedding', 'lm_head'.
A part is constructed from `PartSpec.params` (keyword arguments) on the CPU, without
touching a device; it declares its tensors with `param_specs()` (local name ->
ParamSpec) and receives them, already on the device and in their kept dtype, through
`bind()`.  No part knows which model it is in.

  Norm.forward(ctx, x, out=None, delta=None, row_idx=None) -> Tensor
      x: the float32 residual stream [T, h]; if `delta` is given it is added into x
      first (a norm with `adds_partial_sums` also takes a stack [S, T, h] of partial
      sums).  Returns the normalised rows in the activation dtype.  A norm with
      `leaves_row_scale` takes `scaled_ok=True` from a block whose reader has
      `takes_row_scaled`, and may then return a RowScaled instead: rows that still
      lack their scalar factor, which the reader's first product applies.
  PositionEncoding.apply(ctx, q, k, positions) -> None          (in place, generic path)
      q [T, QH, d], k [T, KH, d].  A mixer may ask `fused_rotary()` for (inv_freq,
      rotated_width) and apply the rotation inside its own kernel instead.
  Mixer.forward(ctx, xn, residual, cache) -> None | Tensor
      xn: normalised input [T, h] in the activation dtype; the mixer ADDS its output
      into `residual` (float32 [T, h]) - or, when `ctx.defer_residual` is set, may
      return what is still to be added ([T, h] or a stack [S, T, h]) for the next norm.  `cache` is the LayerCache of the layer
      (parts/context.py).  `cache_spec()` / `state_spec()` say what the layer needs
      from the cache manager: paged keys/values and/or a fixed-size state per request.
  FeedForward.forward(ctx, xn, residual) -> None | Tensor        (same convention)
  Block.forward(ctx, x, cache[, delta]) -> None | Tensor         (x updated in place; a block with
      `hands_on_sums` takes what the block before left to be added and returns its own)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional, Tuple

import torch

from ..weights.params import ParamSpec
from .spec import PartSpec


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values of every token (or of the last `window` tokens) in pages."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class SlotStateSpec:
    """A state of fixed size per live request, zeroed when the request is admitted."""
    shape: Tuple[int, ...]
    dtype: str = "float32"                      # "float32" or "act" (the activation dtype)


@dataclass
class RowScaled:
    """Rows that still lack a scalar factor each: row t stands for
    rows[t] / sqrt(sum(sumsq[t]) / width + eps) - an RMS norm whose division is left to the product
    that reads the rows, which multiplies its results by the factor (ops.gemm_bf16(..., row_scale=))."""
    rows: torch.Tensor                  # [T, h] bfloat16: x * weight
    sumsq: torch.Tensor                 # [T, parts] float32: the sum of x^2 by chunks of columns
    width: int
    eps: float

    @property
    def shape(self):
        return self.rows.shape

    @property
    def dtype(self):
        return self.rows.dtype

    @property
    def device(self):
        return self.rows.device

    def scale(self):
        return (self.sumsq, self.width, self.eps)


@dataclass
class PreparedRows:
    """What a product that added into the residual stream made for the norm that reads the stream next: that norm's
    rows without their factor.  Handed on in the place of a sum still to be added; only `norm` can take it."""
    norm: object
    rows: torch.Tensor                  # [T, h] bfloat16: the new residual * the norm's weight
    sumsq: torch.Tensor                 # [T, parts] float32


class Part:
    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """`tensors`: local name -> device tensor, for every name of param_specs() that
        the checkpoint (or an optional tensor's fallback) supplied."""


class Norm(Part):
    def forward(self, ctx, x, out=None, delta=None, row_idx=None):
        raise NotImplementedError


class PositionEncoding(Part):
    def apply(self, ctx, q, k, positions) -> None:
        raise NotImplementedError

    def fused_rotary(self):
        """(inv_freq float32 device tensor [rot/2], rot) if this encoding is a plain
        rotation of pairs (p, p+rot/2) by pos*inv_freq[p], else None."""
        return None

    def table_key(self):
        """A hashable value that is equal for two encodings exactly when they make the same per-step table
        from the same positions: layers with equal keys share one table a step.  The default shares nothing."""
        return ("position", id(self))

    def prepare(self, device) -> None:
        """Build device-side tables (called once, after the weights are bound)."""


class Mixer(Part):
    # A mixer with a state_spec() may set this if its step over single-token entries takes the slots from
    # ctx.entry_slot (the device table) and nothing about the batch from the host mirrors (ctx.slots, ctx.q_start,
    # ...): decode-only steps are then replayed from a captured CUDA graph, whose padding rows point at a slot
    # that belongs to no request.  Otherwise a model with such a mixer runs every step eagerly.
    steps_from_device_tables = False

    # Optional: decode_plan(live, largest_tiles, total_tiles) -> hashable.  What a decode step fixes beyond its shapes
    # (the attention: its key splits) for that many requests and 64-key tiles.  The engine asks the first mixer that
    # has it, keys its captured steps by the answer and hands it back as ctx.decode_plan.

    def cache_spec(self) -> Optional[PagedKVSpec]:
        return None

    def state_spec(self) -> Optional[SlotStateSpec]:
        return None

    def prepare(self, device, dtype) -> None:
        pass

    def forward(self, ctx, xn, residual, cache) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, xn, residual) -> None:
        raise NotImplementedError


_REGISTRY: Dict[Tuple[str, str], Callable[..., Any]] = {}


def register_part(category: str, kind: str, factory: Callable[..., Any]) -> None:
    """Register `factory(**params)` under (category, kind).  Re-registering replaces."""
    _REGISTRY[(category, kind)] = factory


def unregister_part(category: str, kind: str) -> None:
    _REGISTRY.pop((category, kind), None)


def build_part(category: str, spec: PartSpec):
    _ensure_builtin()
    try:
        factory = _REGISTRY[(category, spec.kind)]
    except KeyError:
        known = sorted(k for c, k in _REGISTRY if c == category)
        raise KeyError(f"no {category} part of kind '{spec.kind}' is registered (known: {known})") from None
    return factory(**dict(spec.params))


_done = False


def _ensure_builtin() -> None:
    global _done
    if _done:
        return
    _done = True
    from . import norm, rope, attention, ffn, embedding, block  # noqa: F401  (each registers itself)
