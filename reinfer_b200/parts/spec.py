"""A model as data.  An architecture's `build_spec(config)` returns a `ModelSpec`:
which part (by registered kind, with its sizes and constants as parameters) sits
where in which layer, under which tensor-name prefix, and in which order the layers
run.  Nothing here knows a model's name; `parts/model.py` turns it into objects.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    kind: str                                   # key in the registry of its category
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""                            # tensor names of the part are prefix + local name


@dataclass(frozen=True)
class LayerSpec:
    name: str                                   # unique; also the default tensor prefix of the layer
    mixer: PartSpec
    ffn: PartSpec
    mixer_norm: PartSpec
    ffn_norm: PartSpec
    block: str = "prenorm"                      # arrangement of the four parts (registry 'block')
    cache_from: Optional[str] = None            # read (and do not write) the cache of that layer


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    final_norm: PartSpec
    lm_head: PartSpec
    order: Tuple[int, ...] = ()                 # indices into `layers` in run order; () = each once
    ignorable_tensors: Tuple[str, ...] = ()     # names a checkpoint may hold beyond the expected ones

    def run_order(self) -> Tuple[int, ...]:
        return self.order if self.order else tuple(range(len(self.layers)))
