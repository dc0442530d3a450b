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


def role_category(role: str) -> str:
    """The registry category of a layer's part, read off its role's name: 'mixer' -> mixer, 'ffn' -> ffn,
    any role that ends in 'norm' -> norm.  A role of another name states its category itself."""
    if role == "mixer" or role.endswith("_mixer"):
        return "mixer"
    if role == "ffn" or role.endswith("_ffn"):
        return "ffn"
    if role.endswith("norm"):
        return "norm"
    raise ValueError(f"role '{role}' does not tell its category: give it as (category, PartSpec)")


class LayerSpec:
    """A layer: a name, the block arrangement (registry 'block'), and the parts that the arrangement
    works with, each under a role of the arrangement's choosing.

        LayerSpec("l3", block="prenorm", mixer=..., ffn=..., mixer_norm=..., ffn_norm=...)
        LayerSpec("l4", block="my_sandwich", mixer=..., ffn=..., pre_mixer_norm=..., post_mixer_norm=..., ...)
        LayerSpec("l5", block="my_gate", mixer=..., gate=("ffn", PartSpec(...)))

    Roles are keyword arguments: a PartSpec (category read off the role's name, see `role_category`)
    or a pair (category, PartSpec).  `parts` maps role -> (category, PartSpec) in the order given.
    Which roles there must be is the block's business, not the framework's: a layer with four norms,
    with mixer and feed-forward side by side, or without a feed-forward needs a block class and no
    change here.  At most one part of a layer is a mixer (the part that owns a cache)."""

    def __init__(self, name: str, block: str = "prenorm", cache_from: Optional[str] = None, **roles):
        self.name = name                            # unique; also the default tensor prefix of the layer
        self.block = block
        self.cache_from = cache_from                # read (and do not write) the cache of that layer
        parts: Dict[str, Tuple[str, PartSpec]] = {}
        for role, value in roles.items():
            if isinstance(value, PartSpec):
                parts[role] = (role_category(role), value)
            else:
                category, spec = value
                if not isinstance(spec, PartSpec):
                    raise TypeError(f"layer {name}: role '{role}' needs a PartSpec or (category, PartSpec)")
                parts[role] = (str(category), spec)
        if sum(1 for c, _ in parts.values() if c == "mixer") > 1:
            raise ValueError(f"layer {name}: more than one mixer; give the second a layer of its own")
        self.parts = parts

    def __getattr__(self, role: str) -> PartSpec:
        parts = self.__dict__.get("parts", {})
        if role in parts:
            return parts[role][1]
        raise AttributeError(role)

    def __repr__(self) -> str:
        return f"LayerSpec({self.name!r}, block={self.block!r}, roles={list(self.parts)})"


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
