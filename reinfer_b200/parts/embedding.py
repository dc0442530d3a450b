"""Token embedding (a row gather into the float32 residual stream) and the output
head (final norm on the wanted rows only, then the vocabulary product in float32,
never rounded: crates/cuda/src/engine.rs:4337-4347).  The reference computes the
head for every prompt row and keeps the last (engine.rs:5685-5720); here only the
rows whose logits are asked for are normalised and multiplied."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import Part, register_part
from .linear import matmul


class Embedding(Part):
    def __init__(self, vocab: int, hidden: int):
        self.vocab, self.hidden = int(vocab), int(hidden)
        self.weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab, self.hidden), init="table")}

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, ctx) -> torch.Tensor:
        x = torch.empty((ctx.n_tokens, self.hidden), dtype=torch.float32, device=ctx.device)
        ops.embed_gather(self.weight, ctx.token_ids, x, ctx.slot_token, ctx.entry_slot, ctx.tok_entry)
        return x


class LMHead(Part):
    """`tied`: the embedding table is the output matrix; the model hands it over in bind()
    under the local name 'weight' either way."""

    def __init__(self, vocab: int, hidden: int, tied: bool = False, fallback: str = ""):
        self.vocab, self.hidden, self.tied, self.fallback = int(vocab), int(hidden), bool(tied), fallback
        self.weight = None

    def param_specs(self):
        if self.tied:
            return {}
        return {"weight": ParamSpec((self.vocab, self.hidden), optional=bool(self.fallback), fallback=self.fallback)}

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, ctx, xn_rows: torch.Tensor) -> torch.Tensor:
        return matmul(ctx, xn_rows, self.weight, out_dtype=torch.float32)


register_part("embedding", "embedding", Embedding)
register_part("lm_head", "linear", LMHead)
