"""Typed configuration of the Qwen3 dense architecture.

Keys, defaults and validation follow the reference's parser
(crates/arch/src/llama.rs:304-396): `max_position_embeddings`,
`num_hidden_layers`, `hidden_size`, `intermediate_size`, `vocab_size` and
`num_attention_heads` are required; `num_key_value_heads` defaults to the query
head count; `head_dim` defaults to hidden/heads; `rope_theta` defaults to 1e6 for
this family (llama.rs:50-55); `rms_norm_eps` defaults to 1e-5 (llama.rs:371-372).
The reference silently ignores `attention_bias`, `rope_scaling`,
`use_sliding_window` and `hidden_act`; here a value of one of them that would
change the arithmetic is refused, because a silently different model is worse
than an error.  Per-head q/k RMSNorm is a property of the architecture name
(llama.rs:315), not a key.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Mapping, Optional, Tuple

from .errors import InvalidValue, MissingKey


def _uint(d: Mapping[str, Any], key: str, *, required: bool = True, default=None) -> int:
    v = d.get(key)
    if v is None:
        if required:
            raise MissingKey(key)
        return default
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise InvalidValue(key, f"expected a non-negative integer, got {v!r}")
    return int(v)


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rope_theta: float = 1e6
    rms_norm_eps: float = 1e-5
    tie_word_embeddings: bool = False
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Qwen3ForCausalLM"

    # the family's end-of-sequence id where neither generation_config.json nor config.json
    # names one (crates/arch/src/llama.rs:423-431)
    default_eos_ids = (151645,)

    # ---- parsing ---------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen3Config":
        ctx = _uint(d, "max_position_embeddings")
        n_layer = _uint(d, "num_hidden_layers")
        hidden = _uint(d, "hidden_size")
        inter = _uint(d, "intermediate_size")
        vocab = _uint(d, "vocab_size")
        qh = _uint(d, "num_attention_heads")
        for key, val in (("max_position_embeddings", ctx), ("num_hidden_layers", n_layer),
                         ("hidden_size", hidden), ("intermediate_size", inter),
                         ("vocab_size", vocab)):
            if val == 0:
                raise InvalidValue(key, "must be > 0")
        if qh == 0:
            raise InvalidValue("num_attention_heads", "query head count must be > 0")
        kvh = _uint(d, "num_key_value_heads", required=False, default=qh)
        if kvh == 0 or kvh > qh:
            raise InvalidValue("num_key_value_heads", "kv heads must be in 1..=query heads")
        if qh % kvh != 0:
            # The reference accepts this and truncates the ratio (llama.rs:343-348);
            # the result is a model nobody trained, so it is refused here.
            raise InvalidValue("num_key_value_heads",
                               f"query heads ({qh}) must be a multiple of kv heads ({kvh})")
        head_dim = _uint(d, "head_dim", required=False, default=None)
        if head_dim is None:
            head_dim = hidden // qh if hidden % qh == 0 else 0
        if head_dim == 0:
            raise InvalidValue("head_dim", "cannot derive head_dim from hidden_size/head_count")
        if head_dim % 2 != 0:
            raise InvalidValue("head_dim", "rotary encoding pairs (p, p+d/2): head_dim must be even")
        theta = d.get("rope_theta", 1e6)
        if isinstance(theta, bool) or not isinstance(theta, (int, float)) \
                or not math.isfinite(theta) or theta <= 0:
            raise InvalidValue("rope_theta", "rope theta must be finite and > 0")
        eps = d.get("rms_norm_eps", 1e-5)
        if isinstance(eps, bool) or not isinstance(eps, (int, float)) \
                or not math.isfinite(eps) or eps < 0:
            raise InvalidValue("rms_norm_eps", "must be finite and >= 0")
        # keys that would change the arithmetic if honoured
        if d.get("attention_bias"):
            raise InvalidValue("attention_bias", "projections with bias are not part of this architecture")
        if d.get("rope_scaling") not in (None, {}):
            raise InvalidValue("rope_scaling", "scaled rotary variants are not implemented")
        if d.get("use_sliding_window"):
            raise InvalidValue("use_sliding_window", "sliding-window layers are not part of this architecture")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise InvalidValue("hidden_act", f"only 'silu' is implemented, got {act!r}")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (int(eos),)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(int(e) for e in eos)
        else:
            raise InvalidValue("eos_token_id", "expected an integer or a list of integers")
        bos = d.get("bos_token_id")
        archs = d.get("architectures")
        name = archs[0] if isinstance(archs, list) and archs else "Qwen3ForCausalLM"
        return cls(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter,
                   num_hidden_layers=n_layer, num_attention_heads=qh,
                   num_key_value_heads=kvh, head_dim=head_dim,
                   max_position_embeddings=ctx, rope_theta=float(theta),
                   rms_norm_eps=float(eps),
                   tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
                   bos_token_id=bos if isinstance(bos, int) else None,
                   eos_token_ids=eos_ids, architecture=name)

    def to_dict(self) -> dict:
        """The config.json form of this configuration (what random-weights mode writes)."""
        out = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
        }
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            out["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                   else list(self.eos_token_ids))
        return out
