"""What a step hands to the parts: the flat batch of tokens with its per-token and
per-entry tables on the device, and each layer's slice of the cache.

Entries are the (request, next tokens) pairs of the step, decode entries (one token)
first.  All device tables are int32.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Tuple, Dict, List, Optional

import torch


@dataclass
class GroupView:
    """One cache group (layers with the same paged-cache needs) during a step."""
    page_size: int
    block_table: torch.Tensor          # [n_entries, max_pages] page ids; -1 where no page is held
    kv_slot: torch.Tensor              # [n_tokens] page*page_size+offset where each new token is stored
    max_pages: int
    window: Optional[int]


@dataclass
class LayerCache:
    """What one layer sees of the cache."""
    kv: Optional[torch.Tensor] = None  # [num_pages, 2, kv_heads, page_size, head_dim] of the layer it reads
    group: Optional[GroupView] = None
    write: bool = True                 # False: the layer reads another layer's cache and stores nothing
    state: Optional[torch.Tensor] = None   # [num_slots, *shape] fixed-size state, row = request slot


@dataclass
class StepContext:
    dtype: torch.dtype                 # activation dtype (float32 or bfloat16)
    device: torch.device
    n_tokens: int
    n_entries: int
    n_decode: int                      # leading entries that bring exactly one token
    token_ids: torch.Tensor            # [T]
    positions: torch.Tensor            # [T] absolute position of each token
    tok_entry: torch.Tensor            # [T] entry index (= block-table row) of each token
    cu_q: torch.Tensor                 # [E+1] first token of each entry
    kv_len: torch.Tensor               # [E] tokens of the request after this step
    entry_slot: torch.Tensor           # [E] request slot (row of fixed-size states)
    want_slot: Optional[torch.Tensor] = None   # [R] the slot of the request behind each wanted row
    slot_token: Optional[torch.Tensor] = None  # [slots] the token last drawn for each slot's request (token id < 0: take this)
    # host mirrors
    q_start: List[int] = field(default_factory=list)      # E+1
    start_pos: List[int] = field(default_factory=list)    # E
    slots: List[int] = field(default_factory=list)        # E
    max_q_len: int = 0
    max_kv_len: int = 0
    decode_kv_tiles: Optional[Tuple[int, int]] = None     # (sum, largest) of the decode entries' 64-key tiles; None: all as max_kv_len
    decode_plan: Optional[object] = None                  # what the mixer's decode_plan() answered for this step (a captured step is made for one)
    layer_caches: Dict[str, LayerCache] = field(default_factory=dict)
    shared: Dict[object, torch.Tensor] = field(default_factory=dict)   # what one layer computed for all (per step)
    defer_residual: bool = False       # parts may return what is to be added to the residual; the next norm adds it
    # The norm that reads the residual stream next, named by a block (or the model's loop) where the part that runs now
    # may do that norm's work in its last product and hand its rows on instead of a sum (`matmul_into_residual`);
    # None: nobody asked.  `norm_after_block`: the same for the last part of a block, set by the loop over the layers.
    norm_ahead: Optional[object] = None
    norm_after_block: Optional[object] = None

    def empty(self, shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)
