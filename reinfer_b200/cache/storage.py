"""The device memory behind the cache manager: for each group one array
`[layers, 1 + pages + 1, 2 (k, v), kv_heads, page_size, head_dim]` (a layer's slice
without its first and last page is what its kernels get; inside a page the layout is
head-major, so the keys of one (page, head) are one dense `[page_size, head_dim]` tile;
the two pages around a layer's own are guard bands: they hold a fixed pattern that no
kernel may touch, `check_guards` looks at them), and for each layer with a
fixed-size state one array `[slots + 1, *shape]` (the last row is nobody's); and the
slots' own rows: last token, sampler record, recent tokens (the reference keeps these on
the host, bin/reinfer/src/sched_loop.rs:464-485, and only transient `[B]` rows on the
device, crates/cuda/src/engine.rs:1854-1875).
(The reference keeps one f16 buffer, K region then V region, layer folded into the
page index: crates/cuda/src/decode.rs:664-698.)
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .manager import CacheManager


SLOT_RECORD_BYTES = 64          # sizeof(RbSampleParams); the sampler checks it against the library
SLOT_HISTORY = 64               # tokens of the penalty window a slot can hold
GUARD_PATTERN = 0x5A5A          # every 16 bits of a guard page


class CacheStorage:
    def __init__(self, manager: CacheManager, dtype: torch.dtype, device):
        self.manager = manager
        self.dtype = dtype
        self.device = torch.device(device)
        self.group_arrays: List[torch.Tensor] = []
        self.layer_kv: Dict[str, torch.Tensor] = {}
        for g in manager.groups:
            arr = torch.zeros((len(g.layers), g.pool.total + 2, 2, g.spec.kv_heads, manager.page_size, g.spec.head_dim),
                              dtype=dtype, device=self.device)
            for edge in (0, g.pool.total + 1):
                arr[:, edge].view(torch.int16).fill_(GUARD_PATTERN)
            self.group_arrays.append(arr)
            for li, name in enumerate(g.layers):
                self.layer_kv[name] = arr[li, 1:g.pool.total + 1]          # page -1 and page `total` are the guards
        self.layer_state: Dict[str, torch.Tensor] = {}
        for name, spec in manager.states.items():
            sdt = dtype if spec.dtype == "act" else getattr(torch, spec.dtype)
            # one row more than there are slots: the last row belongs to nobody (padding rows of a captured
            # decode step point at it, so that they disturb no request's state)
            self.layer_state[name] = torch.zeros((manager.max_seqs + 1,) + tuple(spec.shape), dtype=sdt, device=self.device)
        self.inert_slot = manager.max_seqs
        # the request slots' own rows (as many, plus nobody's): the token last drawn for the request, the sampler's
        # record (parameters, seed, count of draws: csrc/sampler.cu RbSampleParams) and its ring of recent tokens.
        # The sampler kernel reads and writes them; the host writes a row when a request is admitted.
        self.slot_token = torch.zeros(manager.max_seqs + 1, dtype=torch.int32, device=self.device)
        self.slot_records = torch.zeros((manager.max_seqs + 1, SLOT_RECORD_BYTES), dtype=torch.uint8, device=self.device)
        self.slot_history = torch.zeros((manager.max_seqs + 1, SLOT_HISTORY), dtype=torch.int32, device=self.device)

    def check_guards(self) -> List[str]:
        """The guard pages that no longer hold their pattern, as "layer name: before|after" (empty: all intact).
        A page index of -1 or of the pool's size that reached a store would show here.  Synchronises; for tests
        and for looking into a fault, not for every step."""
        bad = []
        for g, arr in zip(self.manager.groups, self.group_arrays):
            for which, edge in (("before", 0), ("after", g.pool.total + 1)):
                touched = (arr[:, edge].reshape(len(g.layers), -1).view(torch.int16) != GUARD_PATTERN).any(dim=1).tolist()
                bad += [f"{name}: {which}" for name, t in zip(g.layers, touched) if t]
        return bad

    def zero_slot(self, slot: int) -> None:
        """A fixed-size state starts at zero when its request is admitted."""
        for t in self.layer_state.values():
            t[slot].zero_()

    def bytes(self) -> int:
        return sum(a.numel() * a.element_size() for a in self.group_arrays) + \
            sum(a.numel() * a.element_size() for a in self.layer_state.values())

    @staticmethod
    def bytes_per_page(manager_groups, page_size: int, dtype: torch.dtype) -> int:
        isz = torch.empty((), dtype=dtype).element_size()
        return sum(len(g.layers) * 2 * g.spec.kv_heads * page_size * g.spec.head_dim * isz for g in manager_groups)
