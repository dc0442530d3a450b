"""A model built from a `ModelSpec`: embedding, layers (each a block over the parts its
spec names by role), final norm, output head, and the order in which layers run.  The class knows no
architecture; everything it does is driven by the spec.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Tuple

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import PagedKVSpec, SlotStateSpec, _REGISTRY, _ensure_builtin, build_part
from .spec import LayerSpec, ModelSpec, PartSpec


class Layer:
    """The parts of one layer, built from its spec, and the block that arranges them."""

    def __init__(self, spec: LayerSpec):
        self.spec = spec
        self.name = spec.name
        self.parts_by_role = {role: build_part(category, pspec) for role, (category, pspec) in spec.parts.items()}
        mixers = [self.parts_by_role[r] for r, (c, _) in spec.parts.items() if c == "mixer"]
        self.mixer = mixers[0] if mixers else None           # the part that owns a cache, if the layer has one
        self.norms = [self.parts_by_role[r] for r, (c, _) in spec.parts.items() if c == "norm"]
        _ensure_builtin()
        try:
            block_cls = _REGISTRY[("block", spec.block)]
        except KeyError:
            raise KeyError(f"no block arrangement '{spec.block}' is registered") from None
        self.block = block_cls(self.parts_by_role)

    def __getattr__(self, role: str):
        parts = self.__dict__.get("parts_by_role", {})
        if role in parts:
            return parts[role]
        raise AttributeError(role)

    def parts(self):
        return tuple((pspec, self.parts_by_role[role]) for role, (_, pspec) in self.spec.parts.items())

    def cache_spec(self):
        return self.mixer.cache_spec() if self.mixer is not None else None

    def state_spec(self):
        return self.mixer.state_spec() if self.mixer is not None else None


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = build_part("embedding", spec.embedding)
        self.layers: List[Layer] = [Layer(ls) for ls in spec.layers]
        names = [l.name for l in self.layers]
        if len(set(names)) != len(names):
            raise ValueError("layer names must be unique")
        self.final_norm = build_part("norm", spec.final_norm)
        self.lm_head = build_part("lm_head", spec.lm_head)
        self.order = spec.run_order()
        self._chain = ops.StreamChain()         # what the streaming kernels of a pass read, in order (for their L2 hints)
        for i in self.order:
            if not 0 <= i < len(self.layers):
                raise ValueError(f"run order names layer {i} of {len(self.layers)}")
        # a layer that runs more than once has a cache (pages, state) of its own for every run:
        # run k of layer `name` uses the cache key `name` (first run) or `name#k`
        seen: Dict[int, int] = {}
        self.run: List[Tuple[int, str]] = []
        for i in self.order:
            k = seen.get(i, 0)
            seen[i] = k + 1
            self.run.append((i, self.layers[i].name if k == 0 else f"{self.layers[i].name}#{k}"))
        # sums may be left for the next norm only if every norm can add a stack of partial sums and every
        # block hands on what its parts leave
        norms = [n for l in self.layers for n in l.norms] + [self.final_norm]
        self._norms_add_partial_sums = all(getattr(n, "adds_partial_sums", False) for n in norms) and \
            all(getattr(l.block, "hands_on_sums", False) for l in self.layers) and ops.DEFER_SUMS
        by_name = {l.name: l for l in self.layers}
        for l in self.layers:
            src = l.spec.cache_from
            if src is not None:
                if src not in by_name:
                    raise ValueError(f"layer {l.name} reads the cache of unknown layer {src}")
                if by_name[src].spec.cache_from is not None:
                    raise ValueError(f"layer {l.name} reads the cache of {src}, which has none of its own")
                if by_name[src].cache_spec() != l.cache_spec():
                    raise ValueError(f"layer {l.name} and {src} need different caches")

    # ---- tensors -------------------------------------------------------------
    def _all_parts(self):
        s = self.spec
        yield s.embedding, self.embedding
        for l in self.layers:
            yield from l.parts()
        yield s.final_norm, self.final_norm
        yield s.lm_head, self.lm_head

    def param_specs(self) -> Dict[str, ParamSpec]:
        out: Dict[str, ParamSpec] = {}
        for pspec, part in self._all_parts():
            for local, ps in part.param_specs().items():
                name = pspec.prefix + local
                if name in out and out[name] != ps:
                    raise ValueError(f"tensor {name} is declared twice with different specs")
                out[name] = ps
        return out

    def bind(self, state: Mapping[str, torch.Tensor]) -> None:
        """Hand every part its tensors.  An optional tensor that is absent is replaced by its
        fallback (another global name); a tied output head gets the embedding table."""
        for pspec, part in self._all_parts():
            local: Dict[str, torch.Tensor] = {}
            for name, ps in part.param_specs().items():
                g = pspec.prefix + name
                if g in state:
                    local[name] = state[g]
                elif ps.optional and ps.fallback and ps.fallback in state:
                    local[name] = state[ps.fallback]
                elif not ps.optional:
                    raise KeyError(f"tensor {g} was not loaded")
            if part is self.lm_head and getattr(part, "tied", False):
                local["weight"] = state[self.spec.embedding.prefix + "weight"]
            part.bind(local)

    def prepare(self, device, dtype) -> None:
        for l in self.layers:
            if l.mixer is not None:
                l.mixer.prepare(device, dtype)

    # ---- what the cache manager has to provide -------------------------------
    def cache_layout(self):
        """(paged, states): paged maps each cache key (a run of a layer) that owns pages to its
        PagedKVSpec; states maps each key with a fixed-size state to its SlotStateSpec.  Layers
        that read another layer's cache own no pages."""
        paged: Dict[str, PagedKVSpec] = {}
        states: Dict[str, SlotStateSpec] = {}
        for i, key in self.run:
            l = self.layers[i]
            cs, ss = l.cache_spec(), l.state_spec()
            if cs is not None and l.spec.cache_from is None:
                paged[key] = cs
            if ss is not None:
                states[key] = ss
        return paged, states

    def cache_bindings(self):
        """For every run: (cache key, key of the pages it reads or None, whether it stores into them)."""
        out = []
        for i, key in self.run:
            l = self.layers[i]
            if l.cache_spec() is None:
                out.append((key, None, False))
            elif l.spec.cache_from is not None:
                out.append((key, l.spec.cache_from, False))
            else:
                out.append((key, key, True))
        return out

    # ---- the forward pass of one step ------------------------------------------
    def forward(self, ctx, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the step's tokens through every layer in run order; return float32 logits
        [len(want_rows), vocab] for the wanted token rows (None if none are wanted)."""
        ctx.shared.clear()                      # what layers share is computed anew in every pass (a captured pass included)
        previous = ops.set_chain(self._chain)   # the streaming kernels learn from the last pass what they may prefetch
        self._chain.begin()
        try:
            x = self.embedding.forward(ctx)
            ctx.defer_residual = self._norms_add_partial_sums
            delta = None                        # what a block left to be added to x by the norm that reads x next
            for n, (i, key) in enumerate(self.run):
                block = self.layers[i].block
                if self._norms_add_partial_sums:
                    # the block that runs next may let this one's last product do its first norm's work
                    nxt = self.layers[self.run[n + 1][0]].block if n + 1 < len(self.run) else None
                    entry = getattr(nxt, "entry_norm", None) if getattr(nxt, "hands_on_sums", False) else None
                    ctx.norm_after_block = entry() if entry is not None else None
                    delta = block.forward(ctx, x, ctx.layer_caches[key], delta)
                else:
                    block.forward(ctx, x, ctx.layer_caches[key])
            ctx.norm_after_block = None
            if want_rows is None or want_rows.numel() == 0:
                return None                     # (a sum still owed to x is dropped with x)
            xn = self.final_norm.forward(ctx, x, delta=delta, row_idx=want_rows)
            logits = self.lm_head.forward(ctx, xn)
            self._chain.end()                   # a pass that came this far is complete
            return logits
        finally:
            self._chain.live = False
            ops.set_chain(previous)


def expected_params(spec: ModelSpec) -> Dict[str, ParamSpec]:
    """Tensor names and shapes of a spec (parts are built on the CPU; no device is touched)."""
    return Model(spec).param_specs()
