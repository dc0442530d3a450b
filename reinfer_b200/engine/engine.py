"""The engine: a model, its cache, and ONE step function.

`step(entries)` takes a batch of (request, its next tokens, the places among them whose
logits are wanted): portions of prompts beside single decoded tokens, cut anywhere.  It
runs only those tokens, as one batch, against what earlier steps left in the cache, and
returns float32 logits on the device for the wanted places, in the order of the entries
and of their `want` lists.  The reference has three separate calls for this and cannot
continue a prompt (crates/cuda/src/engine.rs:3739 `step`, :5218 `prefill_batch`, :5853
`batch_decode_step`; bin/reinfer/src/sched_loop.rs:188-195); here one launch sequence
serves every composition of the batch.

Everything the kernels need to know about the batch goes to the device as one int32
block per step (token ids, positions, entry of each token, per-entry tables, and per
cache group the store slots and the block tables), staged in pinned memory.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import gc
import numpy as np
import torch

from .. import ops
from ..cache import CacheManager, CacheStorage, OutOfPages
from ..hostio import PinnedRing
from ..config.registry import load_config, resolve_architecture
from ..parts.context import GroupView, LayerCache, StepContext
from ..parts.model import Model
from ..weights.loader import load_state, random_state


class EngineError(RuntimeError):
    pass


class KernelWaitTimeout(EngineError):
    """A kernel gave up a bounded wait and left its output unfinished."""


class EmbeddingOov(EngineError):
    """A token id outside the vocabulary, refused before any launch
    (crates/cuda/src/engine.rs:3784-3786)."""


FROM_SLOT = -1      # in place of a token id: "the token that the sampler drew for this request in the step before"


@dataclass
class StepEntry:
    request_id: Hashable
    tokens: Sequence[int]                    # ids; a single FROM_SLOT for a live request whose last draw the host has not read yet
    want: Sequence[int] = ()                 # indices into `tokens`


_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
           "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


def parse_dtype(d) -> torch.dtype:
    if isinstance(d, torch.dtype):
        if d not in (torch.float32, torch.bfloat16):
            raise EngineError(f"dtype {d}: the engine runs in float32 or bfloat16")
        return d
    try:
        return _DTYPES[str(d).lower()]
    except KeyError:
        raise EngineError(f"dtype {d!r}: expected float32 or bfloat16") from None


class Engine:
    """Built from a model folder (`from_model_dir`) or from a configuration with random
    weights made on the device (`from_config`)."""

    def __init__(self, config, spec, state: Dict[str, torch.Tensor], dtype: torch.dtype, *,
                 page_size: int = 64, num_pages: Optional[int] = None, max_tokens: Optional[int] = None,
                 max_num_seqs: int = 64, device="cuda:0", memory_fraction: float = 0.9,
                 cuda_graphs: bool = True, consume_state: bool = False):
        """consume_state: the dictionary of tensors may be emptied once the parts hold what they need (the parts
        concatenate some of them; the originals would else stay alive beside the copies)."""
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        ops.require_device()
        self.config = config
        self.dtype = dtype
        self.model = Model(spec)
        self.model.bind(state)
        if consume_state:
            state.clear()
            torch.cuda.empty_cache()            # what the copies replaced goes back to the driver before memory is counted
        self.model.prepare(self.device, dtype)
        self.vocab_size = spec.vocab_size
        paged, states = self.model.cache_layout()
        self.page_size = int(page_size)
        if num_pages is None:
            if max_tokens is not None:
                num_pages = max(1, -(-int(max_tokens) // self.page_size))
            else:
                num_pages = self._pages_from_memory(paged, memory_fraction, max_num_seqs)
        self.cache = CacheManager(paged, states, self.page_size, int(num_pages), int(max_num_seqs))
        self.storage = CacheStorage(self.cache, dtype, self.device)
        self._staging = PinnedRing()
        ops.status_word()                       # binds the kernels' error word to host memory (before any capture)
        self._undo = None                       # the cache manager's snapshot from before the step in progress
        # What the owner of the engine hangs onto a step (the sampler does): `on_admit(request_id, slot)` when a
        # request gets its slot; `epilogue(logits, want_slot, rows)` after the forward pass, on the same stream,
        # with the slot of the request behind each wanted row - inside the captured graph for decode-only steps.
        self.on_admit = None
        self._epilogue = None
        self.steps_run = 0
        # decode-only steps replay a captured CUDA graph per (batch bucket, block-table width, the mixers' plan).  Padding rows
        # point at a slot that belongs to nobody.  A mixer with state takes part only if it says that its
        # single-token step reads the batch from the device tables alone (`steps_from_device_tables`): what
        # it read from the host mirrors would be frozen into the capture.
        stateful = [l.mixer for l in self.model.layers if l.mixer is not None and l.mixer.state_spec() is not None]
        self.cuda_graphs = bool(cuda_graphs) and all(getattr(m, "steps_from_device_tables", False) for m in stateful)
        self._graphs: Dict[tuple, "_DecodeGraph"] = {}
        self._graph_pool = None
        self.graph_replays = 0
        # the first mixer that can say what a decode step fixes beyond its shapes (Mixer.decode_plan); None: nobody can
        self._planner = next((l.mixer.decode_plan for l in self.model.layers
                              if l.mixer is not None and callable(getattr(l.mixer, "decode_plan", None))), None)

    @property
    def epilogue(self):
        return self._epilogue

    @epilogue.setter
    def epilogue(self, fn) -> None:
        if fn is not self._epilogue:
            self._graphs.clear()                # captured steps hold the old epilogue's launches
        self._epilogue = fn

    # ---- construction ---------------------------------------------------------------
    @classmethod
    def from_model_dir(cls, model_dir: str, dtype="bfloat16", device="cuda:0", **kw) -> "Engine":
        dt = parse_dtype(dtype)
        arch, config = load_config(model_dir)
        spec = arch.build_spec(config)
        expected = Model(spec).param_specs()
        state = load_state(model_dir, expected, dt, torch.device(device), ignorable=spec.ignorable_tensors)
        return cls(config, spec, state, dt, device=device, consume_state=True, **kw)

    @classmethod
    def from_config(cls, config, seed: int = 0, dtype="bfloat16", device="cuda:0", **kw) -> "Engine":
        """Random weights drawn on the device (no files): for measurements at full size."""
        dt = parse_dtype(dtype)
        arch = resolve_architecture(config.to_dict())
        spec = arch.build_spec(config)
        expected = Model(spec).param_specs()
        state = random_state(expected, seed, dt, torch.device(device))
        return cls(config, spec, state, dt, device=device, consume_state=True, **kw)

    def _pages_from_memory(self, paged, fraction: float, max_num_seqs: int) -> int:
        """pages = floor((fraction * total - in use) / bytes per page)
        (crates/memory/src/budget.rs:99-155)."""
        from ..cache.manager import group_layers
        isz = 4 if self.dtype == torch.float32 else 2
        per_page = sum(len(n) * 2 * s.kv_heads * self.page_size * s.head_dim * isz for s, n in group_layers(paged))
        if per_page == 0:
            return 1
        free, total = torch.cuda.mem_get_info(self.device)
        # what is still to come besides the cache: the sampler's scratch rows and a captured step's logits (a row of
        # vocabulary floats per request each), the products' workspace, and the activations of the largest step
        rows = -(-int(max_num_seqs) // 8) * 8
        reserve = 3 * rows * self.vocab_size * 4 + (4 << 30)
        budget = int(total * fraction) - (total - free) - reserve
        n = budget // per_page
        if n < 1:
            raise EngineError("no memory left for the cache after the weights")
        return int(n)

    # ---- the step ----------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], logits: bool = True) -> Optional[torch.Tensor]:
        """Runs the entries' tokens as one batch and returns the logits at the wanted places (None if
        none is wanted; with logits=False a caller whose epilogue has used them says that it does not
        need them, which saves a decode step the copy out of its graph's buffer).  If anything fails after the cache manager was changed (a kernel wrapper that
        refuses its arguments, a launch error), the admissions and reservations of this step are undone
        before the error goes on: every request is as it was before the call.  A kernel whose bounded
        wait gave up in an earlier step makes this call raise before it launches anything
        (`check_status`)."""
        self.check_status()
        entries = [e for e in entries if len(e.tokens) > 0]
        try:
            if self.cuda_graphs and entries and len(entries) <= MAX_GRAPH_BATCH and all(len(e.tokens) == 1 for e in entries):
                return self._step_graph(entries, logits)
            ctx, want_rows, lens_after = self._prepare(entries)
            if ctx is None:
                return None
            out = self.model.forward(ctx, want_rows)
            if out is not None and self._epilogue is not None:
                self._epilogue(out, ctx.want_slot, out.shape[0])
        except BaseException:
            self._rollback()
            raise
        self._undo = None
        for rid, n in lens_after:
            self.cache.commit(rid, n)
        self.steps_run += 1
        return out

    def _rollback(self) -> None:
        undo, self._undo = self._undo, None
        if undo is not None:
            self.cache.restore(undo)

    def check_status(self) -> None:
        """Raise if a kernel's bounded wait has given up (crates/cuda/src/engine.rs:3697-3737 `BarrierTimeout`,
        :3849-3897 `SyncTimeout` are the reference's form of it).  The word lives in host memory that the
        kernels write to, so this costs one load; it is complete for every step whose results the host has
        already waited for (the sampled tokens, a copy of the logits).  After the error: `clear_status`."""
        code = ops.status_word()
        if code:
            raise KernelWaitTimeout(f"{ops.describe_status(code)} (status word 0x{code:x}); the logits of that step "
                                    f"and what it stored in the cache are not to be trusted")

    def clear_status(self) -> int:
        return ops.clear_status()

    def _graph_key(self, entries: Sequence[StepEntry]):
        B = len(entries)
        bucket = B if B <= 8 else -(-B // 8) * 8
        need_pages = 1
        for e in entries:
            cur = self.cache.length(e.request_id) if e.request_id in self.cache else 0
            need_pages = max(need_pages, self.cache.pages_for(cur + 1))
        width = 8
        while width < need_pages:
            width *= 2
        # how full the batch's block tables are, in eighths: requests of unequal lengths want their keys split
        # over more CTAs than the longest alone would suggest, and a captured step keeps the split it was made with
        total = sum(-(-((self.cache.length(e.request_id) if e.request_id in self.cache else 0) + 1) // 64) for e in entries)
        widest = max(1, width * self.page_size // 64)
        fill = min(FILL_STEPS, max(1, (2 * FILL_STEPS * total + B * widest) // (2 * B * widest)))
        # what the mixers fix beyond the shapes (the attention: its key splits) is asked for the requests there are, not
        # for the rows of their bucket - 18 requests want another split than 24 - and for their keys as they are, to
        # an eighth of the widest table; batches with the same answer share a captured step
        plan = None
        if self._planner is not None:
            tiles = max(B, B * widest * fill // FILL_STEPS)
            plan = self._planner(B, widest, tiles)
        return bucket, width, plan if plan is not None else fill

    def _step_graph(self, entries: Sequence[StepEntry], logits: bool = True) -> Optional[torch.Tensor]:
        """A step of single tokens only: fill the graph's static tables and replay it."""
        key = self._graph_key(entries)
        host, lens_after = self._prepare(entries, fixed=key)
        rows = [k for k, e in enumerate(entries) if len(e.want) > 0] if logits else []
        return self._replay(key, host, lens_after, rows, len(entries))

    def _replay(self, key, host, lens_after, rows, B) -> Optional[torch.Tensor]:
        g = self._graphs.pop(key, None)
        if g is None:
            while len(self._graphs) >= MAX_GRAPHS:      # the one replayed longest ago goes (its memory returns to the pool)
                self._graphs.pop(next(iter(self._graphs)))
            g = _DecodeGraph(self, key[0], key[1], key[2])
        self._graphs[key] = g                           # most recently used last
        self._staging.upload(host, self.device, into=g.meta)
        g.graph.replay()
        self.graph_replays += 1
        self._undo = None
        for rid, n in lens_after:
            self.cache.commit(rid, n)
        self.steps_run += 1
        if not rows:
            return None
        # a copy: the graph's own buffer is overwritten by the next replay
        return g.logits[:B].clone() if rows == list(range(B)) else g.logits[rows]

    # ---- one step ahead -----------------------------------------------------------------------
    def prepare_ahead(self, request_ids: Sequence[Hashable]):
        """While the step just launched still runs on the device: build the tables of the NEXT step under
        the guess that exactly these requests go on with one token each (pages are reserved now; the token
        ids are not known yet).  Returns a handle for `step_ahead`, or None if that step cannot be a
        graph replay or the pages are short (the ordinary path then decides what happens)."""
        if not self.cuda_graphs or not request_ids or len(request_ids) > MAX_GRAPH_BATCH:
            return None
        entries = [StepEntry(rid, [0], [0]) for rid in request_ids]
        if any(rid not in self.cache for rid in request_ids):
            return None
        key = self._graph_key(entries)
        try:
            host, lens_after = self._prepare(entries, fixed=key)
        except OutOfPages:
            return None
        self._undo = None                               # the pages stay with their requests whatever comes of the handle
        return (key, tuple(request_ids), host, lens_after)

    def step_ahead(self, ahead, tokens: Optional[Sequence[int]] = None, logits: bool = True) -> Optional[torch.Tensor]:
        """Run the step prepared by `prepare_ahead`: with the token ids that have arrived since, or
        (tokens=None) with every request's token taken from its slot on the device, where the sampler of
        the step before has left it - then the host need not have seen that step's result at all."""
        key, rids, host, lens_after = ahead
        if tokens is None:
            host[:len(rids)] = FROM_SLOT                # the block starts with the token ids (Engine._layout)
        else:
            for t in tokens:
                if not 0 <= int(t) < self.vocab_size:
                    raise EmbeddingOov(f"token id {t} outside the vocabulary of {self.vocab_size}")
            host[:len(rids)] = tokens
        self.check_status()
        return self._replay(key, host, lens_after, list(range(len(rids))) if logits else [], len(rids))

    def check_guards(self) -> None:
        """Raises if a guard page beside a layer's cache pages no longer holds its pattern (a store reached a page
        index of -1 or of the pool's size).  Synchronises the device: for tests and for looking into a fault."""
        bad = self.storage.check_guards()
        if bad:
            raise EngineError("guard pages of the cache were written: " + ", ".join(bad))

    def finish(self, request_id) -> None:
        """The request is over: its pages and its slot are given back."""
        if request_id in self.cache:
            self.cache.release(request_id)

    def _prepare(self, entries: Sequence[StepEntry], fixed=None):
        """Checks, page reservation and the step's int32 block.  With `fixed` = (entries, block-table
        width) the block has that fixed layout (rows beyond the real entries are inert: no key is
        read or stored for them) and is returned on the host, for a captured graph."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return None, None, []
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise EngineError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if len(e.tokens) == 1:
                lo_t = hi_t = int(e.tokens[0])
                if lo_t == FROM_SLOT and e.request_id in self.cache and self.cache.length(e.request_id) > 0:
                    lo_t = hi_t = 0                     # taken from the request's slot by the embedding
            else:
                arr = np.asarray(e.tokens)
                lo_t, hi_t = int(arr.min()), int(arr.max())
            if lo_t < 0 or hi_t >= self.vocab_size:
                raise EmbeddingOov(f"request {e.request_id!r}: token id {lo_t if lo_t < 0 else hi_t} outside the "
                                   f"vocabulary of {self.vocab_size}")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise EngineError(f"request {e.request_id!r}: wanted place {w} outside its {len(e.tokens)} tokens")
        cm = self.cache
        # enough slots and pages for the whole batch, before anything is changed
        new = [e for e in entries if e.request_id not in cm]
        if len(new) > cm.free_slots():
            raise OutOfPages(f"{len(new)} new requests but {cm.free_slots()} free slots")
        need = 0
        for e in entries:
            cur = cm.length(e.request_id) if e.request_id in cm else 0
            have = len(cm.table(e.request_id, 0)) if (e.request_id in cm and cm.groups) else 0
            need += max(0, cm.pages_for(cur + len(e.tokens)) - have)
        if need > cm.free_pages():
            raise OutOfPages(f"the step needs {need} more pages, {cm.free_pages()} are free")
        self._undo = cm.snapshot([e.request_id for e in entries])     # from here on the manager changes
        for e in new:
            slot = cm.admit(e.request_id)
            self.storage.zero_slot(slot)
            if self.on_admit is not None:
                self.on_admit(e.request_id, slot)
        # decode entries first, each kind in the order given
        order = sorted(range(len(entries)), key=lambda i: (len(entries[i].tokens) != 1, i))
        internal = [entries[i] for i in order]
        E = len(internal)
        q_len = [len(e.tokens) for e in internal]
        start = [cm.length(e.request_id) for e in internal]
        for e, s, n in zip(internal, start, q_len):
            cm.reserve(e.request_id, s + n)
        q_start = np.zeros(E + 1, dtype=np.int64)
        np.cumsum(q_len, out=q_start[1:])
        T = int(q_start[-1])
        n_decode = sum(1 for n in q_len if n == 1)
        slots = [cm.slot(e.request_id) for e in internal]
        # wanted rows in the caller's order
        pos_in_internal = {id(e): k for k, e in enumerate(internal)}
        want_rows = [int(q_start[pos_in_internal[id(e)]]) + int(w) for e in entries for w in e.want]
        R = len(want_rows)

        n_groups = len(cm.groups)
        max_pages = [max(1, max(len(cm.table(e.request_id, g)) for e in internal)) for g in range(n_groups)]
        E_real, T_real = E, T
        if fixed is not None:
            E = T = R = fixed[0]
            max_pages = [fixed[1]] * n_groups
            want_rows = list(range(R))
        off, cur = self._layout(T, E, R, max_pages)
        host = np.zeros(cur, dtype=np.int32)

        def sec(name):
            o, n = off[name]
            return host[o:o + n]

        tok, pos, ent = sec("token_ids"), sec("positions"), sec("tok_entry")
        ent[:] = np.arange(T, dtype=np.int32) if fixed is not None else 0
        for k, e in enumerate(internal):
            a, b = int(q_start[k]), int(q_start[k + 1])
            tok[a:b] = np.asarray(e.tokens, dtype=np.int32)
            pos[a:b] = np.arange(start[k], start[k] + q_len[k], dtype=np.int32)
            ent[a:b] = k
        if fixed is not None:
            sec("cu_q")[:] = np.arange(E + 1, dtype=np.int32)
        else:
            sec("cu_q")[:] = q_start
        sec("kv_len")[:E_real] = np.asarray(start) + np.asarray(q_len)
        sec("entry_slot")[:] = self.storage.inert_slot
        sec("entry_slot")[:E_real] = slots
        if R:
            sec("want_rows")[:] = want_rows
            ws = sec("want_slot")
            ws[:] = self.storage.inert_slot
            if fixed is None:
                ws[:] = [slots[pos_in_internal[id(e)]] for e in entries for _ in e.want]
            else:                                       # row k is entry k; an entry that wants nothing draws for nobody
                for k, e in enumerate(internal):
                    if len(e.want) > 0:
                        ws[k] = slots[k]
        for g in range(n_groups):
            ks = sec(f"kv_slot{g}")
            ks[:] = -1
            bt = sec(f"block_table{g}").reshape(E, max_pages[g])
            bt[:] = -1
            for k, e in enumerate(internal):
                table = cm.table_array(e.request_id, g)
                bt[k, :table.shape[0]] = table
                a, b = int(q_start[k]), int(q_start[k + 1])
                if b - a == 1:
                    p0 = start[k]
                    page = int(table[p0 // self.page_size])
                    if page < 0:
                        raise EngineError(f"request {e.request_id!r}: position {p0} lies in a page that was given back")
                    ks[a] = page * self.page_size + p0 % self.page_size
                else:
                    ks[a:b] = cm.write_slots(e.request_id, g, start[k], q_len[k])
        lens_after = [(e.request_id, s + n) for e, s, n in zip(internal, start, q_len)]
        if fixed is not None:
            return host, lens_after
        dev = self._staging.upload(host, self.device)
        ctx = self._context(dev, off, T, E, n_decode, max_pages, [int(v) for v in q_start], list(start), slots,
                            max(q_len), max(s + n for s, n in zip(start, q_len)))
        if n_decode:
            tiles = [-(-(s + 1) // 64) for s in start[:n_decode]]
            ctx.decode_kv_tiles = (sum(tiles), max(tiles))
        o, n = off["want_rows"]
        return ctx, (dev[o:o + n] if R else None), lens_after

    @staticmethod
    def _layout(T: int, E: int, R: int, max_pages):
        """Offsets (in int32 elements, 16-byte aligned sections) of the step's block."""
        off = {}
        cur = 0

        def take(name, n):
            nonlocal cur
            off[name] = (cur, n)
            cur += (n + 3) // 4 * 4

        take("token_ids", T); take("positions", T); take("tok_entry", T)
        take("cu_q", E + 1); take("kv_len", E); take("entry_slot", E); take("want_rows", max(R, 1)); take("want_slot", max(R, 1))
        for g in range(len(max_pages)):
            take(f"kv_slot{g}", T); take(f"block_table{g}", E * max_pages[g])
        return off, cur

    def _context(self, dev: torch.Tensor, off, T: int, E: int, n_decode: int, max_pages, q_start, start, slots,
                 max_q_len: int, max_kv_len: int) -> StepContext:
        """Views of the device block as the tables the parts read, and each layer's cache."""
        cm = self.cache

        def dsec(name):
            o, n = off[name]
            return dev[o:o + n]

        views = []
        for g, grp in enumerate(cm.groups):
            views.append(GroupView(page_size=self.page_size,
                                   block_table=dsec(f"block_table{g}").view(E, max_pages[g]),
                                   kv_slot=dsec(f"kv_slot{g}"), max_pages=max_pages[g], window=grp.window))
        layer_caches: Dict[str, LayerCache] = {}
        for key, src, write in self.model.cache_bindings():
            lc = LayerCache(write=write)
            if src is not None and src in cm.group_of_layer:
                lc.kv = self.storage.layer_kv[src]
                lc.group = views[cm.group_of_layer[src]]
            if key in self.storage.layer_state:
                lc.state = self.storage.layer_state[key]
            layer_caches[key] = lc
        return StepContext(dtype=self.dtype, device=self.device, n_tokens=T, n_entries=E, n_decode=n_decode,
                           token_ids=dsec("token_ids"), positions=dsec("positions"), tok_entry=dsec("tok_entry"),
                           cu_q=dsec("cu_q"), kv_len=dsec("kv_len"), entry_slot=dsec("entry_slot"),
                           want_slot=dsec("want_slot"), slot_token=self.storage.slot_token,
                           q_start=q_start, start_pos=start, slots=slots, max_q_len=max_q_len, max_kv_len=max_kv_len,
                           layer_caches=layer_caches)


MAX_GRAPH_BATCH = 256
MAX_GRAPHS = 24                         # captured decode steps kept at a time (one per batch bucket, block-table width and plan in use)
FILL_STEPS = 8                          # the keys in a batch's block tables are counted to so many eighths of the widest table


class _DecodeGraph:
    """A captured decode step for `batch` single-token entries and block tables `width` pages wide.
    Its tables live in `meta` (a static int32 block the engine refills before every replay); its
    logits [batch, vocab] in `logits`."""

    def __init__(self, engine: "Engine", batch: int, width: int, plan=None):
        n_groups = len(engine.cache.groups)
        off, total = Engine._layout(batch, batch, batch, [width] * n_groups)
        host = np.zeros(total, dtype=np.int32)
        for name, (o, n) in off.items():
            if name.startswith("kv_slot") or name.startswith("block_table"):
                host[o:o + n] = -1                       # inert rows: nothing stored, nothing read
        o, n = off["tok_entry"]; host[o:o + n] = np.arange(batch)
        o, n = off["cu_q"]; host[o:o + n] = np.arange(batch + 1)
        o, n = off["want_rows"]; host[o:o + n] = np.arange(batch)
        inert = engine.storage.inert_slot
        o, n = off["entry_slot"]; host[o:o + n] = inert
        o, n = off["want_slot"]; host[o:o + n] = inert
        self.meta = torch.from_numpy(host).to(engine.device)
        ctx = engine._context(self.meta, off, batch, batch, batch, [width] * n_groups, list(range(batch + 1)),
                              [0] * batch, [inert] * batch, 1, width * engine.page_size)
        widest = max(1, width * engine.page_size // 64)
        if engine._planner is not None:
            ctx.decode_plan = plan                          # the third part of the key is the mixers' plan
        else:
            fill = plan if plan is not None else FILL_STEPS # without a planner it is the tables' fill in eighths
            ctx.decode_kv_tiles = (max(batch, batch * widest * fill // FILL_STEPS), widest)
        o, n = off["want_rows"]
        want = self.meta[o:o + n]
        def run():
            logits = engine.model.forward(ctx, want)
            if engine._epilogue is not None:
                engine._epilogue(logits, ctx.want_slot, batch)
            return logits

        l0 = ops.launches
        run()                                            # eager once: lazy set-up must not fall into the capture
        self.n_launches = ops.launches - l0              # kernels of this library in one replay
        torch.cuda.synchronize()
        if engine._graph_pool is None:
            engine._graph_pool = torch.cuda.graph_pool_handle()
        self.graph = torch.cuda.CUDAGraph()
        # Nothing may free device or pinned memory while a stream captures (the capture is then invalid, and the next
        # launch says so).  Python's collector can: an engine that the program dropped earlier - its graphs, their
        # pool, its pinned buffers - is garbage with cycles and goes whenever the collector next runs.  So it runs
        # now, and not again before the capture has ended.
        was_enabled = gc.isenabled()
        gc.collect()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph, pool=engine._graph_pool):
                self.logits = run()
        finally:
            if was_enabled:
                gc.enable()
