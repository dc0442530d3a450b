"""The one registry from an architecture's name to its configuration class and
its model description.

The reference resolves the name with a hard-coded `match` on
`architectures[0]`, else `model_type` (crates/arch/src/llama.rs:305-317).  Here
it is a table that anybody may extend: an entry holds the typed configuration
class (parsed from config.json's own keys) and a function that turns such a
configuration into a `ModelSpec` (reinfer_b200/parts/spec.py), i.e. into data
that names the parts of every layer.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional, Tuple

from .errors import MissingKey, UnknownArchitecture


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: Any                       # has from_dict(mapping) and to_dict()
    build_spec: Callable[[Any], Any]      # config -> parts.spec.ModelSpec
    aliases: Tuple[str, ...] = ()


_REGISTRY: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls, build_spec, aliases=()) -> Architecture:
    """Add (or replace) an architecture.  `aliases` are further names, such as the
    `model_type` string, that resolve to the same entry."""
    arch = Architecture(name, config_cls, build_spec, tuple(aliases))
    _REGISTRY[name] = arch
    for a in arch.aliases:
        _REGISTRY[a] = arch
    return arch


def unregister_architecture(name: str) -> None:
    arch = _REGISTRY.pop(name, None)
    if arch is not None:
        for a in arch.aliases:
            _REGISTRY.pop(a, None)


def registered_architectures():
    return sorted({a.name for a in _REGISTRY.values()})


def architecture_name(config: Mapping[str, Any]) -> str:
    """`architectures[0]`, else `model_type` (llama.rs:305-311)."""
    archs = config.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    mt = config.get("model_type")
    if isinstance(mt, str):
        return mt
    raise MissingKey("architectures")


def resolve_architecture(config: Mapping[str, Any]) -> Architecture:
    _ensure_builtin()
    name = architecture_name(config)
    arch = _REGISTRY.get(name)
    if arch is None:
        raise UnknownArchitecture(name, registered_architectures())
    return arch


def load_config(model_dir: str):
    """Read `model_dir/config.json`; return (architecture entry, typed config)."""
    path = os.path.join(model_dir, "config.json")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    arch = resolve_architecture(raw)
    return arch, arch.config_cls.from_dict(raw)


def resolve_eos(config, model_dir: Optional[str] = None) -> Tuple[int, ...]:
    """End-of-sequence ids.  Order of sources as in the reference
    (llama.rs:406-432): generation_config.json, then config.json, then the
    fallback ids of the architecture's family, which its configuration class
    states as `default_eos_ids`.  A list-valued `eos_token_id` stops on every id
    of the list (the reference keeps only the first)."""
    if model_dir is not None:
        gpath = os.path.join(model_dir, "generation_config.json")
        if os.path.exists(gpath):
            with open(gpath, "r", encoding="utf-8") as f:
                g = json.load(f)
            e = g.get("eos_token_id")
            if isinstance(e, int) and not isinstance(e, bool):
                return (e,)
            if isinstance(e, list) and e:
                return tuple(int(x) for x in e)
    ids = tuple(getattr(config, "eos_token_ids", ()) or ())
    if ids:
        return ids
    return tuple(getattr(config, "default_eos_ids", ()) or ())


_builtin_done = False


def _ensure_builtin() -> None:
    global _builtin_done
    if _builtin_done:
        return
    _builtin_done = True
    from ..models import qwen3 as _q  # registers itself on import
    _q.register()
