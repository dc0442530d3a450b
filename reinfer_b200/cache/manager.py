"""The cache manager: who holds which page, on the host, without any device call.

Keys and values live in pages of `page_size` tokens.  Layers with the same needs
(kv heads, head size, window) form a group; a group has its own pool of page ids and
every live request has one block table per group, which all layers of the group share
(a page id indexes each layer's own array).  A request also holds one slot: the row of
every fixed-size per-request state and of the sampler's per-request data.

Pages come from a LIFO free stack (the reference's `PagePool`, crates/memory/src/pool.rs:
61-155; its serving path hands out whole contiguous windows per request instead,
crates/memory/src/segment.rs:258-347) one at a time as a request grows; they go back
when the request ends (in reverse order of acquisition, so reuse is deterministic) or,
in a group with a window, as soon as no later token can attend to them.

Invariants (checked by `check()` and by the tests): for each group, pages in use + pages
free = total; no page is in two block tables or twice in one; nothing is freed twice.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np

from ..parts.base import PagedKVSpec, SlotStateSpec


class OutOfPages(RuntimeError):
    """Not enough free pages (or no free slot) for what was asked; nothing was changed."""


class CacheError(RuntimeError):
    """A misuse of the manager: unknown request, double free, shrinking a request."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a pool needs at least one page")
        self.total = int(num_pages)
        self._free: List[int] = list(range(self.total - 1, -1, -1))    # pop() gives 0 first
        self._held = [False] * self.total
        self.allocs = 0
        self.frees = 0

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def in_use(self) -> int:
        return self.total - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        p = self._free.pop()
        self._held[p] = True
        self.allocs += 1
        return p

    def free(self, page: int) -> None:
        if not 0 <= page < self.total or not self._held[page]:
            raise CacheError(f"page {page} is freed but not held")
        self._held[page] = False
        self._free.append(page)
        self.frees += 1

    def check(self) -> None:
        assert self.in_use + self.free_count == self.total
        assert self.allocs - self.frees == self.in_use
        assert len(set(self._free)) == len(self._free), "a page is twice in the free stack"
        assert all(not self._held[p] for p in self._free)


@dataclass
class CacheGroup:
    spec: PagedKVSpec
    layers: Tuple[str, ...]
    pool: PagePool

    @property
    def window(self) -> Optional[int]:
        return self.spec.window


@dataclass
class _Seq:
    slot: int
    length: int = 0                                     # tokens whose keys are cached (committed)
    reserved: int = 0                                   # tokens that pages are held for (>= length)
    tables: List[List[int]] = field(default_factory=list)   # per group: page id per page index, -1 = given back
    np_tables: List[np.ndarray] = field(default_factory=list)   # the same as int32 arrays (capacity grows by doubling)


def group_layers(paged: Dict[str, PagedKVSpec]) -> List[Tuple[PagedKVSpec, Tuple[str, ...]]]:
    """Layers with equal needs share a group, in order of first appearance."""
    groups: Dict[PagedKVSpec, List[str]] = {}
    for name, spec in paged.items():
        groups.setdefault(spec, []).append(name)
    return [(s, tuple(n)) for s, n in groups.items()]


class CacheManager:
    def __init__(self, paged: Dict[str, PagedKVSpec], states: Dict[str, SlotStateSpec],
                 page_size: int, num_pages: int, max_seqs: int):
        if page_size <= 0 or max_seqs <= 0:
            raise ValueError("page_size and max_seqs must be positive")
        self.page_size = int(page_size)
        self.max_seqs = int(max_seqs)
        self.groups: List[CacheGroup] = [CacheGroup(s, n, PagePool(num_pages)) for s, n in group_layers(paged)]
        self.group_of_layer: Dict[str, int] = {n: gi for gi, g in enumerate(self.groups) for n in g.layers}
        self.states = dict(states)
        self._free_slots: List[int] = list(range(self.max_seqs - 1, -1, -1))
        self._seqs: Dict[Hashable, _Seq] = {}

    # ---- queries -----------------------------------------------------------------
    def __contains__(self, rid) -> bool:
        return rid in self._seqs

    def live(self) -> List[Hashable]:
        return list(self._seqs)

    def length(self, rid) -> int:
        return self._seq(rid).length

    def slot(self, rid) -> int:
        return self._seq(rid).slot

    def free_slots(self) -> int:
        return len(self._free_slots)

    def free_pages(self) -> int:
        """Free pages of the tightest group (every group has to hold a request's tokens)."""
        return min((g.pool.free_count for g in self.groups), default=1 << 30)

    def total_pages(self) -> int:
        return min((g.pool.total for g in self.groups), default=1 << 30)

    def table(self, rid, group: int) -> List[int]:
        return self._seq(rid).tables[group]

    def table_array(self, rid, group: int) -> np.ndarray:
        """The block table as an int32 array (a view: valid until the request grows)."""
        s = self._seq(rid)
        return s.np_tables[group][:len(s.tables[group])]

    def _seq(self, rid) -> _Seq:
        try:
            return self._seqs[rid]
        except KeyError:
            raise CacheError(f"request {rid!r} is not live") from None

    def _first_needed_page(self, g: CacheGroup, next_pos: int) -> int:
        """Index of the first page that a token at position >= next_pos can still read."""
        if g.window is None:
            return 0
        return max(0, next_pos - g.window + 1) // self.page_size

    def pages_needed(self, rid, new_len: int) -> int:
        """Most pages any group has to add so that the request can hold `new_len` tokens."""
        s = self._seq(rid)
        need_idx = (new_len + self.page_size - 1) // self.page_size
        return max((max(0, need_idx - len(t)) for t in s.tables), default=0)

    def pages_for(self, n_tokens: int) -> int:
        return (n_tokens + self.page_size - 1) // self.page_size

    # ---- life of a request -----------------------------------------------------------
    def admit(self, rid) -> int:
        """Give the request a slot (and empty block tables); returns the slot."""
        if rid in self._seqs:
            raise CacheError(f"request {rid!r} is already live")
        if not self._free_slots:
            raise OutOfPages("no free request slot")
        slot = self._free_slots.pop()
        self._seqs[rid] = _Seq(slot=slot, tables=[[] for _ in self.groups],
                               np_tables=[np.full(16, -1, dtype=np.int32) for _ in self.groups])
        return slot

    def reserve(self, rid, new_len: int) -> None:
        """Hold pages in every group for tokens up to `new_len`.  All or nothing."""
        s = self._seq(rid)
        if new_len < s.length:
            raise CacheError(f"request {rid!r} cannot shrink from {s.length} to {new_len}")
        need_idx = (new_len + self.page_size - 1) // self.page_size
        for g, t in zip(self.groups, s.tables):
            if need_idx - len(t) > g.pool.free_count:
                raise OutOfPages(f"request {rid!r} needs {need_idx - len(t)} more pages, "
                                 f"{g.pool.free_count} are free")
        for gi, (g, t) in enumerate(zip(self.groups, s.tables)):
            if len(t) < need_idx:
                arr = s.np_tables[gi]
                if arr.shape[0] < need_idx:
                    grown = np.full(max(need_idx, 2 * arr.shape[0]), -1, dtype=np.int32)
                    grown[:len(t)] = arr[:len(t)]
                    s.np_tables[gi] = arr = grown
                while len(t) < need_idx:
                    p = g.pool.alloc()
                    arr[len(t)] = p
                    t.append(p)
        s.reserved = max(s.reserved, new_len)

    def commit(self, rid, new_len: int) -> None:
        """The step has stored tokens up to `new_len`; pages that a window has passed go back."""
        s = self._seq(rid)
        cap = min((len(t) for t in s.tables), default=None)
        if new_len < s.length or (cap is not None and new_len > cap * self.page_size):
            raise CacheError(f"request {rid!r}: commit of {new_len} tokens outside what is reserved")
        s.length = new_len
        for gi, (g, t) in enumerate(zip(self.groups, s.tables)):
            if g.window is None:
                continue
            first = min(self._first_needed_page(g, new_len), len(t))
            for i in range(first):
                if t[i] >= 0:
                    g.pool.free(t[i])
                    t[i] = -1
                    s.np_tables[gi][i] = -1

    def release(self, rid) -> None:
        """The request ends: every page (latest first) and the slot go back."""
        s = self._seqs.pop(rid, None)
        if s is None:
            raise CacheError(f"request {rid!r} is released but not live")
        for g, t in zip(self.groups, s.tables):
            for p in reversed(t):
                if p >= 0:
                    g.pool.free(p)
        self._free_slots.append(s.slot)

    # ---- undoing a step that failed ------------------------------------------------------
    def snapshot(self, rids: Sequence[Hashable]):
        """What `restore` needs to undo admissions and reservations made after this moment for these requests
        (commits are not undone: a step commits only after it has run)."""
        snap = {}
        for rid in rids:
            s = self._seqs.get(rid)
            snap[rid] = None if s is None else (s.reserved, [len(t) for t in s.tables])
        return snap

    def restore(self, snap) -> None:
        """Give back what was taken since `snapshot`: a request admitted since then leaves altogether (pages and
        slot); one that was live then keeps the pages it held then and returns the later ones, latest first."""
        for rid, before in snap.items():
            s = self._seqs.get(rid)
            if s is None:
                continue
            if before is None:
                self.release(rid)
                continue
            reserved, lens = before
            for gi, (g, t) in enumerate(zip(self.groups, s.tables)):
                while len(t) > lens[gi]:
                    p = t.pop()
                    s.np_tables[gi][len(t)] = -1
                    if p >= 0:
                        g.pool.free(p)
            s.reserved = max(reserved, s.length)

    # ---- per-step tables ---------------------------------------------------------------
    def write_slots(self, rid, group: int, start: int, n: int) -> List[int]:
        """page*page_size+offset for the tokens at positions start..start+n-1."""
        t = self._seq(rid).tables[group]
        ps = self.page_size
        if n == 1:
            page = t[start // ps]
            if page < 0:
                raise CacheError(f"request {rid!r}: position {start} lies in a page that was given back")
            return [page * ps + start % ps]
        out = []
        for pos in range(start, start + n):
            page = t[pos // ps]
            if page < 0:
                raise CacheError(f"request {rid!r}: position {pos} lies in a page that was given back")
            out.append(page * ps + pos % ps)
        return out

    def check(self) -> None:
        for gi, g in enumerate(self.groups):
            g.pool.check()
            seen = set()
            for rid, s in self._seqs.items():
                for p in s.tables[gi]:
                    if p < 0:
                        continue
                    assert p not in seen, f"page {p} of group {gi} is held twice"
                    seen.add(p)
            assert len(seen) == g.pool.in_use, f"group {gi}: {g.pool.in_use} pages in use, {len(seen)} in tables"
        slots = [s.slot for s in self._seqs.values()]
        assert len(set(slots)) == len(slots)
        assert len(slots) + len(self._free_slots) == self.max_seqs
        assert not (set(slots) & set(self._free_slots))
