"""Sampling options, with the names and meanings of the reference
(`SamplerParams`, crates/kernels/src/sampler_chain.rs:105-155; command-line defaults
bin/reinfer/src/main.rs:246-294)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass
class SamplingParams:
    temperature: float = 0.0              # <= 0: greedy, no random number is consumed
    top_k: int = 0                        # 0 (or >= vocabulary): off
    top_p: float = 1.0                    # <= 0 or >= 1: off
    min_p: float = 0.0                    # <= 0: off; keep prob >= max_prob * min_p
    repeat_penalty: float = 1.0           # > 1 turns it on: l > 0 ? l / r : l * r over the last repeat_last_n tokens
    repeat_last_n: int = 64
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    logit_bias: Tuple[Tuple[int, float], ...] = ()   # (token id, addend) pairs, added to the logits before all else
    seed: Optional[int] = None            # None: derived from the engine's seed and the request's arrival number
    max_tokens: int = 256                 # hard cap of new tokens
    stop_token_ids: Tuple[int, ...] = ()
    stop_sequences: Tuple[Tuple[int, ...], ...] = ()   # token-id sequences; generation stops when one ends the output
    ignore_eos: bool = False

    def validate(self) -> None:
        if self.max_tokens < 0:
            raise ValueError("max_tokens must be >= 0")
        if self.repeat_last_n < 0 or self.repeat_last_n > 64:
            raise ValueError("repeat_last_n must be in 0..64")
        if len(self.logit_bias) > 1024:
            raise ValueError("logit_bias takes at most 1024 entries")
        if len({int(i) for i, _ in self.logit_bias}) != len(self.logit_bias) or any(int(i) < 0 for i, _ in self.logit_bias):
            raise ValueError("logit_bias: token ids must be distinct and non-negative")
        if any(t < 0 for seq in self.stop_sequences for t in seq):
            raise ValueError("stop_sequences: token ids must be non-negative")
        if self.temperature != self.temperature:
            raise ValueError("temperature is NaN")
