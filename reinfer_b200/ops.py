"""Python face of the kernel library: loads the shared library that
`csrc/build.py` builds and wraps each C entry point in a function that takes
torch tensors (as storage only: pointers, shapes and dtypes are read, no torch
operator runs).  Kernels launch on torch's current CUDA stream, so they order with
torch's allocator and can be captured into CUDA graphs.

There is no fallback: without the library, or on a device that is not sm_100,
every call raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_void_p, c_int, c_float, c_longlong, c_char_p
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


_lib = None


def lib():
    """The loaded library (built at the first call if needed)."""
    global _lib
    if _lib is None:
        path = _build.ensure_built()
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the kernel library {path}: {e}") from None
        _lib.rb_last_error.restype = c_char_p
        if _lib.rb_abi_version() != 1:
            raise KernelError("kernel library has another ABI version")
        if os.environ.get("REINFER_B200_GEMM_SCHEDULE"):
            # 0: one CTA per tile, 1: persistent CTAs (default) for prompt portions
            _lib.rb_set_gemm_persistent(int(os.environ["REINFER_B200_GEMM_SCHEDULE"]))
        if os.environ.get("REINFER_B200_GEMM_TOKEN_LANES"):
            # prompt portions: 1 a token per accumulator lane (default), 0 a feature per lane
            _lib.rb_set_gemm_token_lanes(int(os.environ["REINFER_B200_GEMM_TOKEN_LANES"]))
        if os.environ.get("REINFER_B200_GEMM_GATED_STREAM"):
            # the gated pair over 65 .. 128 tokens: 1 the streaming kernel with a token per lane (default), 0 a feature per lane
            _lib.rb_set_gemm_gated_stream(int(os.environ["REINFER_B200_GEMM_GATED_STREAM"]))
        if os.environ.get("REINFER_B200_GEMM_TILE_ROWS"):
            # prompt portions: 256 or 224 weight rows a tile; default chosen per product
            _lib.rb_set_gemm_tile_features(int(os.environ["REINFER_B200_GEMM_TILE_ROWS"]))
        if os.environ.get("REINFER_B200_PDL", "1") == "0":
            _lib.rb_set_pdl(0)          # launch every kernel fully serialised (for comparisons)
    return _lib


_checked_device = False


def require_device() -> None:
    """Fail loudly unless a CUDA device of compute capability 10.x is current."""
    global _checked_device
    if _checked_device:
        return
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: reinfer_b200 runs on a B200 (sm_100a) only and has no CPU path")
    cc = lib().rb_device_cc()
    if cc < 0:
        raise KernelError(f"CUDA error {-cc} while reading the device's compute capability")
    if cc // 10 != 10:
        raise KernelError(f"device has compute capability {cc / 10:.1f}; the kernels are built for sm_100a only")
    _checked_device = True


launches = 0          # kernels of this library launched so far (every wrapper passes through _check)


class SegmentProfiler:
    """CUDA-event times of the launches of a step, by named segment (the idea of the reference's DecodeProfiler
    and PrefillProfiler: cudaEvent pairs around named segments, crates/cuda/src/engine.rs:928-1408, 6675-6975).
    While a profiler is installed (`set_profiler`) every wrapper records an event behind its launch; a launch's
    time is the span from the event before it to its own, so the launches are seen one after the other, without
    the overlap that programmatic dependent launch gives them in a plain run: compare shares, as with a profiler.
    Each wrapper also says what the launch has to compute and to move, which gives achieved FLOP/s and bytes/s."""

    def __init__(self) -> None:
        self.marks = []                                     # (name, flops, bytes, event)
        self.start = None

    def begin(self) -> None:
        self.marks = []
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()

    def mark(self, name: str, flops: float, nbytes: float) -> None:
        if self.start is None:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.marks.append((name, flops, nbytes, ev))

    def summary(self):
        """name -> {"n", "us", "tflops", "gbs"} (synchronises); insertion order = order of first launch."""
        torch.cuda.synchronize()
        out, prev = {}, self.start
        for name, flops, nbytes, ev in self.marks:
            us = prev.elapsed_time(ev) * 1e3
            prev = ev
            d = out.setdefault(name, {"n": 0, "us": 0.0, "flops": 0.0, "bytes": 0.0})
            d["n"] += 1; d["us"] += us; d["flops"] += flops; d["bytes"] += nbytes
        for d in out.values():
            t = max(d["us"], 1e-9) * 1e-6
            d["tflops"] = d.pop("flops") / t / 1e12
            d["gbs"] = d.pop("bytes") / t / 1e9
        return out


_profiler: Optional["SegmentProfiler"] = None


def set_profiler(p: Optional["SegmentProfiler"]) -> Optional["SegmentProfiler"]:
    """Install (or, with None, remove) the profiler that the wrappers report to; returns the previous one."""
    global _profiler
    old, _profiler = _profiler, p
    return old


def _check(rc: int, what: str, flops: float = 0.0, nbytes: float = 0.0) -> None:
    global launches
    launches += 1
    if _profiler is not None and rc == 0:
        _profiler.mark(what, flops, nbytes)
    if rc == 0:
        return
    if rc < 0:
        raise KernelError(f"{what}: {lib().rb_last_error().decode()}")
    raise KernelError(f"{what}: CUDA error {rc} at launch")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """torch's current stream as a raw handle (by torch's own short way where it has one: a step makes hundreds of
    launches and each asks)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not float32 or bfloat16") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


# ------------------------------------------------------------------ wrappers
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, slot_token: Optional[torch.Tensor] = None,
                 entry_slot: Optional[torch.Tensor] = None, tok_entry: Optional[torch.Tensor] = None) -> None:
    """out[t,:] (float32) = table[ids[t],:]; where ids[t] < 0 and the slot tables are given, the id is
    slot_token[entry_slot[tok_entry[t]]]: the token that the sampler left in the request's slot."""
    _need(out.dtype == torch.float32 and ids.dtype == torch.int32, "embed_gather: out float32, ids int32")
    _need(table.is_contiguous() and out.is_contiguous(), "embed_gather: contiguous tensors")
    _check(lib().rb_embed_gather(_p(table), dt(table), _p(ids), _p(slot_token), _p(entry_slot), _p(tok_entry), _p(out),
                                 c_int(ids.numel()), c_int(table.shape[1]), c_int(table.shape[0]), _stream()), "embed_gather")


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, out: torch.Tensor,
                eps: float, row_idx: Optional[torch.Tensor] = None) -> None:
    """x (float32, [rows,h]) += delta if given; out[r] = rmsnorm(x[row_idx[r] or r]) * w.
    delta has x's shape, or one more leading dimension: partial sums [S, rows, h] that are added in
    ascending order (what a split product leaves).  With row_idx the sum is formed for the gathered
    rows only and x itself is left unchanged."""
    _need(x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous(), "rmsnorm: x float32 contiguous")
    h = x.shape[-1]
    rows = out.numel() // h
    n_delta = 0
    if delta is not None:
        _need(delta.is_contiguous() and delta.numel() % x.numel() == 0 and delta.shape[-1] == h, "rmsnorm: delta has x's shape (or a stack of it)")
        n_delta = delta.numel() // x.numel()
    _check(lib().rb_add_rmsnorm(_p(x), _p(delta), c_int(dt(delta) if delta is not None else F32), c_int(n_delta),
                                c_longlong(x.numel()), _p(w), c_int(dt(w)),
                                _p(out), c_int(dt(out)), _p(row_idx), c_int(rows), c_int(h), c_float(eps),
                                _stream()), "add_rmsnorm")


def residual_rowscale(x: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor):
    """x (float32 [rows,h]) += delta (x's shape, or a stack of partial sums added in ascending order); returns
    (y, sumsq): y = bfloat16(x * w) and sumsq [rows, parts] float32, the sum of x^2 by chunks of columns.  The
    product that reads y multiplies its results for row r by 1/sqrt(sum(sumsq[r]) / h + eps): the RMS norm with
    its division moved behind the product (gemm_bf16(..., row_scale=(sumsq, h, eps)))."""
    _need(x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2, "rowscale: x float32 [rows,h] contiguous")
    rows, h = x.shape
    n_delta = 0
    if delta is not None:
        _need(delta.dtype == torch.float32 and delta.is_contiguous() and delta.numel() % x.numel() == 0 and delta.shape[-1] == h,
              "rowscale: delta float32 with x's shape (or a stack of it)")
        n_delta = delta.numel() // x.numel()
    parts = int(lib().rb_rowscale_parts(c_int(h)))
    y = torch.empty((rows, h), dtype=torch.bfloat16, device=x.device)
    sumsq = torch.empty((rows, parts), dtype=torch.float32, device=x.device)
    _check(lib().rb_residual_rowscale(_p(x), _p(delta), c_int(n_delta), c_longlong(x.numel()), _p(w), c_int(dt(w)),
                                      _p(y), _p(sumsq), c_int(rows), c_int(h), _stream()), "residual_rowscale")
    return y, sumsq


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    _need(x.dtype == torch.float32 and x.is_contiguous() and delta.is_contiguous() and x.numel() == delta.numel(),
          "residual_add: x float32, same size")
    _check(lib().rb_residual_add(_p(x), _p(delta), c_int(dt(delta)), c_longlong(x.numel()), _stream()), "residual_add")


def qknorm_rope_append(qkv: torch.Tensor, qw: Optional[torch.Tensor], kw: Optional[torch.Tensor],
                       inv_freq: Optional[torch.Tensor], positions: Optional[torch.Tensor],
                       kv_slot: Optional[torch.Tensor], q_out: torch.Tensor, cache: Optional[torch.Tensor],
                       QH: int, KH: int, d: int, rot: int, page_size: int, eps: float,
                       k_out: Optional[torch.Tensor] = None, cs_table: Optional[torch.Tensor] = None) -> None:
    """Per-head RMSNorm of q and k (if weights are given), rotation of the first `rot` dims (if
    rot > 0), q -> q_out, k and v -> the cache at kv_slot (or k -> k_out, v untouched)."""
    n = qkv.shape[0]
    _need(qkv.is_contiguous() and q_out.is_contiguous(), "qknorm_rope_append: contiguous")
    _need(qkv.shape[-1] == (QH + 2 * KH) * d, "qknorm_rope_append: qkv width")
    wd = dt(qw) if qw is not None else F32
    if qw is not None:
        _need(kw is not None and kw.dtype == qw.dtype, "qknorm_rope_append: q/k norm weights of one dtype")
    _check(lib().rb_qknorm_rope_append(_p(qkv), c_int(dt(qkv)), _p(qw), _p(kw), c_int(wd), _p(inv_freq), _p(cs_table),
                                       _p(positions), _p(kv_slot), _p(q_out), _p(k_out), _p(cache),
                                       c_int(dt(cache) if cache is not None else dt(qkv)),
                                       c_int(n), c_int(QH), c_int(KH), c_int(d), c_int(rot), c_int(page_size),
                                       c_float(eps), _stream()), "qknorm_rope_append")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """(cos, sin) of positions[t] * inv_freq[p] as float32 [T, half, 2]: computed once per step, read by every layer."""
    T, half = positions.numel(), inv_freq.numel()
    cs = torch.empty((T, half, 2), dtype=torch.float32, device=positions.device)
    _check(lib().rb_rope_table(_p(positions), _p(inv_freq), _p(cs), c_int(T), c_int(half), _stream()), "rope_table")
    return cs


def kv_append(k: torch.Tensor, v: torch.Tensor, kv_slot: torch.Tensor, cache: torch.Tensor,
              KH: int, d: int, page_size: int) -> None:
    """k, v: [T, KH*d] views (row stride free, heads contiguous) -> cache pages."""
    _need(k.dtype == v.dtype == cache.dtype, "kv_append: one dtype")
    _need(k.stride(-1) == 1 and v.stride(-1) == 1, "kv_append: rows contiguous")
    _check(lib().rb_kv_append(_p(k), c_longlong(k.stride(0)), _p(v), c_longlong(v.stride(0)), _p(kv_slot), _p(cache),
                              c_int(dt(k)), c_int(k.shape[0]), c_int(KH), c_int(d), c_int(page_size), _stream()),
           "kv_append")


def swiglu(gu: torch.Tensor, out: torch.Tensor) -> None:
    _need(gu.is_contiguous() and out.is_contiguous() and gu.dtype == out.dtype, "swiglu: contiguous, one dtype")
    F_ = out.shape[-1]
    _need(gu.shape[-1] == 2 * F_, "swiglu: input is [gate | up]")
    _check(lib().rb_swiglu(_p(gu), _p(out), c_int(dt(gu)), c_int(out.numel() // F_), c_int(F_), _stream()), "swiglu")


def gemm_ref(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, accumulate: bool = False) -> None:
    """c[M,N] (=|+=) a[M,K] @ w[N,K]^T on the CUDA cores in 32-bit."""
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and tuple(c.shape) == (M, N), "gemm: shapes")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1, "gemm: rows contiguous")
    _check(lib().rb_gemm_ref(_p(a), c_int(dt(a)), _p(w), c_int(dt(w)), _p(c), c_int(dt(c)), c_int(int(accumulate)),
                             c_int(M), c_int(N), c_int(K), c_longlong(a.stride(0)), c_longlong(w.stride(0)),
                             c_longlong(c.stride(0)), _stream()), f"gemm_fma {N}x{K}", 2.0 * M * N * K,
           float(M * K * a.element_size() + N * K * w.element_size() + M * N * c.element_size()))


def paged_attention_ref(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, tok_row: torch.Tensor,
                        positions: torch.Tensor, out: torch.Tensor, QH: int, KH: int, d: int, page_size: int,
                        window: int, scale: float, work=(0.0, 0.0)) -> None:
    _need(q.is_contiguous() and out.is_contiguous() and cache.is_contiguous() and block_table.is_contiguous(),
          "attention: contiguous")
    _need(q.dtype == cache.dtype == out.dtype, "attention: one dtype for q, cache and out")
    _check(lib().rb_paged_attention_ref(_p(q), _p(cache), c_int(dt(q)), _p(block_table), _p(tok_row), _p(positions),
                                        _p(out), c_int(q.shape[0]), c_int(QH), c_int(KH), c_int(d), c_int(page_size),
                                        c_int(block_table.shape[1]), c_int(window), c_float(scale), _stream()),
           "paged_attention_ref", *work)


def fa_group_chunk(group: int) -> int:
    """Query heads of one kv head that share a row tile: the largest divisor of the group up to 16."""
    for c in range(16, 0, -1):
        if group % c == 0:
            return c
    return 1


def fa_decode(q, cache, block_table, cu_q, kv_len, out, first_entry: int, n_entries: int, first_tok: int, n_splits: int,
              QH: int, KH: int, d: int, page_size: int, window: int, scale: float, work=(0.0, 0.0)) -> None:
    """Split-K flash decoding (tensor cores) for entries that bring one token each."""
    part_o = part_lse = None
    if n_splits > 1:
        part_o = torch.empty(n_entries * QH * n_splits * d, dtype=torch.float32, device=q.device)
        part_lse = torch.empty(n_entries * QH * n_splits, dtype=torch.float32, device=q.device)
    _check(lib().rb_fa_decode(_p(q), _p(cache), _p(block_table), _p(cu_q), _p(kv_len), _p(out), _p(part_o), _p(part_lse),
                              c_int(first_entry), c_int(n_entries), c_int(first_tok), c_int(n_splits), c_int(QH), c_int(KH),
                              c_int(d), c_int(page_size), c_int(block_table.shape[1]), c_int(window), c_float(scale),
                              _stream()), "fa_decode", *work)
    if n_splits > 1:
        global launches
        launches += 1                      # the merge kernel


class StreamChain:
    """Which constant ranges (weights) the streaming kernels of one forward pass read, in order.

    A decode step is bound by memory traffic, and memory idles while one product drains and the small
    kernels after it run.  So a streaming kernel (a product over few tokens, decode attention) is told
    which weights the next one reads and calls their first bytes into L2 once its own loads are issued.
    The order is not declared by anyone: every pass writes down what it streamed, and a pass whose
    ranges match the last complete pass step by step learns from it what comes next; after the last
    range comes the first (the next step).  A pass that runs other kernels (a prompt) or another order
    just gets no hint until two passes agree again.
    """

    def __init__(self) -> None:
        self.known: list = []           # (address, bytes) of the last complete pass; bytes == 0: a marker, nothing to fetch
        self.now: list = []
        self.live = False

    def begin(self) -> None:
        self.now = []
        self.live = True

    def end(self) -> None:
        if self.live:
            self.known = self.now
        self.live = False

    def step(self, address: int, nbytes: int):
        """Note that a kernel streams this range now; returns (address, bytes) of what follows, or None."""
        if not self.live:
            return None
        i = len(self.now)
        self.now.append((address, nbytes))
        k = self.known
        if i < len(k) and k[i] == (address, nbytes) and len(k) > 1:
            nxt = k[(i + 1) % len(k)]
            if nxt[1] > 0 and nxt[0] % 16 == 0:
                return nxt
        return None


_chain: Optional[StreamChain] = None
L2_PREFETCH_BYTES = int(float(os.environ.get("REINFER_B200_L2_PREFETCH_MB", "12")) * (1 << 20))
DEFER_SUMS = os.environ.get("REINFER_B200_DEFER_SUMS", "1") != "0"   # split products leave their last sum to the next norm
STREAMING_TOKENS = 64                       # products over at most this many tokens count as weight streaming


def set_chain(chain: Optional[StreamChain]) -> Optional[StreamChain]:
    """Make `chain` the one that the streaming kernels consult (None: no hints); returns the previous one."""
    global _chain
    old, _chain = _chain, chain
    return old


def row_scale_ok(T: int) -> bool:
    """Whether the tensor-core products over T tokens apply the factor of rows that lack it (RowScaled input)."""
    return bool(lib().rb_gemm_row_scale_ok(c_int(int(T))))


def _row_scale_args(row_scale, T: int):
    """(sumsq pointer, parts, width, eps) arguments of a product whose rows still lack their RMS factor."""
    if row_scale is None:
        return c_void_p(0), c_int(0), c_int(0), c_float(0.0)
    sumsq, width, eps = row_scale
    _need(sumsq.dtype == torch.float32 and sumsq.is_contiguous() and sumsq.dim() == 2 and sumsq.shape[0] == T,
          "gemm: row factors come as float32 [tokens, parts]")
    return _p(sumsq), c_int(sumsq.shape[1]), c_int(int(width)), c_float(float(eps))


def _next_range(t: Optional[torch.Tensor], marker: int = 0):
    """(pointer, bytes) arguments of the range that follows tensor t (or the marker) in the active chain."""
    if _chain is None or L2_PREFETCH_BYTES <= 0:
        return c_void_p(0), c_longlong(0)
    nxt = _chain.step(t.data_ptr(), t.numel() * t.element_size()) if t is not None else _chain.step(marker, 0)
    if nxt is None:
        return c_void_p(0), c_longlong(0)
    return c_void_p(nxt[0]), c_longlong(min(nxt[1], L2_PREFETCH_BYTES))


DECODE_SLOTS = 296                          # CTAs of the decode attention that are resident at once (two per SM)
# Clusters merge their splits themselves only while they fill at most this share of the places the device reports: a
# cluster needs its places on one GPC at once, and near the limit clusters wait for one another (measured: 13 splits
# of 16 pairs on 208 of 221 places, 7 splits of 40 pairs on 280 of 296, each 4 % slower a step than a neighbouring count)
CLUSTER_FILL = 0.9
MAX_CLUSTER_SPLITS = 16                     # splits that can merge inside one cluster (more than 8: not portable, asked of the device)
_cluster_slots: dict = {}


def decode_cluster_slots(d: int, n: int) -> int:
    """CTAs of the decode attention that can be resident at once as clusters of n: the fixed figure for portable
    clusters, what the device's occupancy calculation says for larger ones (0: cannot be launched)."""
    if n <= 8:
        return DECODE_SLOTS
    key = (d, n)
    if key not in _cluster_slots:
        _cluster_slots[key] = min(DECODE_SLOTS, int(lib().rb_fa_decode_cluster_slots(c_int(d), c_int(n))))
    return _cluster_slots[key]


def fa_decode_tma(q, cache, block_table, cu_q, kv_len, out, first_entry: int, n_entries: int, first_tok: int, n_splits: int,
                  QH: int, KH: int, d: int, page_size: int, window: int, scale: float, work=(0.0, 0.0)) -> None:
    """Split-K flash decoding with the key/value tiles brought in by TMA (page size a power of two >= 8).
    Up to 16 splits whose CTAs are all resident at once form clusters that merge their results themselves (no scratch,
    no merge kernel); several waves of CTAs, or more splits, go through scratch and the merge kernel (clusters
    that wait for a free place on one GPC were measured slower there)."""
    part_o = part_lse = None
    ctas = n_entries * KH * (QH // KH // fa_group_chunk(QH // KH)) * n_splits
    in_kernel = ATTN_CLUSTER_MERGE and 2 <= n_splits <= min(MAX_CLUSTER_SPLITS, d) and ctas <= CLUSTER_FILL * decode_cluster_slots(d, n_splits)
    if n_splits > 1 and not in_kernel:
        part_o = torch.empty(n_entries * QH * n_splits * d, dtype=torch.float32, device=q.device)
        part_lse = torch.empty(n_entries * QH * n_splits, dtype=torch.float32, device=q.device)
    nw, nb = _next_range(None, marker=cache.data_ptr())
    _check(lib().rb_fa_decode_tma(_p(q), _p(cache), c_longlong(cache.shape[0]), _p(block_table), _p(cu_q), _p(kv_len), _p(out),
                                  _p(part_o), _p(part_lse), c_int(first_entry), c_int(n_entries), c_int(first_tok),
                                  c_int(n_splits), c_int(QH), c_int(KH), c_int(d), c_int(page_size),
                                  c_int(block_table.shape[1]), c_int(window), c_float(scale), nw, nb, _stream()), "fa_decode_tma", *work)


def fa_prefill_tma(q, cache, block_table, cu_q, kv_len, out, first_entry: int, n_entries: int, n_tiles: int,
                   QH: int, KH: int, d: int, page_size: int, window: int, scale: float, work=(0.0, 0.0)) -> None:
    """Paged causal flash attention with the key/value tiles brought in by TMA."""
    _check(lib().rb_fa_prefill_tma(_p(q), _p(cache), c_longlong(cache.shape[0]), _p(block_table), _p(cu_q), _p(kv_len), _p(out),
                                   c_int(first_entry), c_int(n_entries), c_int(n_tiles), c_int(QH), c_int(KH), c_int(d),
                                   c_int(page_size), c_int(block_table.shape[1]), c_int(window), c_float(scale), _stream()),
           "fa_prefill_tma", *work)


def fa_prefill_tc(q, cache, block_table, cu_q, kv_len, out, first_entry: int, n_entries: int, q_lens,
                  QH: int, KH: int, d: int, page_size: int, window: int, scale: float, work=(0.0, 0.0)) -> None:
    """Paged causal flash attention on the tcgen05 tensor cores (scores and the weighted sum in tensor memory):
    head size 128, page size a power of two >= 8.  q_lens: the token counts of the entries (host)."""
    gc = int(lib().rb_fa_prefill_tc_group(c_int(QH), c_int(KH)))
    tpt = int(lib().rb_fa_prefill_tc_rows()) // gc              # tokens that one CTA takes
    n_tiles = sum(-(-int(n) // tpt) for n in q_lens)
    _check(lib().rb_fa_prefill_tc(_p(q), _p(cache), c_longlong(cache.shape[0]), _p(block_table), _p(cu_q), _p(kv_len), _p(out),
                                  c_int(first_entry), c_int(n_entries), c_int(n_tiles), c_int(QH), c_int(KH), c_int(d),
                                  c_int(page_size), c_int(block_table.shape[1]), c_int(window), c_float(scale), _stream()),
           "fa_prefill_tc", *work)


def tma_pages(page_size: int) -> bool:
    return page_size >= 8 and page_size & (page_size - 1) == 0


def fa_prefill(q, cache, block_table, cu_q, kv_len, out, first_entry: int, n_entries: int, n_tiles: int,
               QH: int, KH: int, d: int, page_size: int, window: int, scale: float, work=(0.0, 0.0)) -> None:
    """Paged causal flash attention (tensor cores) for entries that bring several tokens."""
    _check(lib().rb_fa_prefill(_p(q), _p(cache), _p(block_table), _p(cu_q), _p(kv_len), _p(out), c_int(first_entry),
                               c_int(n_entries), c_int(n_tiles), c_int(QH), c_int(KH), c_int(d), c_int(page_size),
                               c_int(block_table.shape[1]), c_int(window), c_float(scale), _stream()), "fa_prefill", *work)


USE_TMA_ATTENTION = os.environ.get("REINFER_B200_TMA_ATTENTION", "1") != "0"
ATTN_CLUSTER_MERGE = os.environ.get("REINFER_B200_ATTN_CLUSTER", "1") != "0"
USE_TC_ATTENTION = os.environ.get("REINFER_B200_TC_ATTENTION", "1") != "0"
MIXED_OVERLAP = os.environ.get("REINFER_B200_MIXED_OVERLAP", "1") != "0"   # decode attention beside the portions' attention
_side_streams: dict = {}


def _side_stream(device) -> "torch.cuda.Stream":
    key = torch.device(device).index or 0
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device)
    return _side_streams[key]
def decode_splits(ctas: int, tiles: int, slots: int = DECODE_SLOTS, head_dim: int = 128, cluster_slots=None,
                  total_tiles: Optional[int] = None) -> int:
    """How many CTAs share one (request, kv head)'s keys: the split count with the least estimated time (ties to
    the smaller).  `ctas` (request, kv head) pairs, the longest of `tiles` 64-key tiles, `total_tiles` over all pairs
    (default: all as long as the longest).  The estimate is fitted to measurements of the kernel at batch 1..64 and
    4k..32k keys, alone and inside whole decode steps:
      - every resident CTA has the first three tiles of its share on their way before the kernels in front of it
        have finished; what is left streams at the memory bandwidth, less what the CTAs' fill and drain cost,
        which weighs the more the fewer tiles a CTA walks:   bytes left / 6.5 TB/s * (1 + 2.7 / tiles per CTA)
      - a CTA alone streams a 64-key tile of 128-wide heads in about a microsecond and needs about five to start
        and finish; the kernel lasts as long as the CTA with most tiles:   (most tiles per CTA - 3) * 1 us + 5 us
        (requests of unequal lengths: the longest alone decides this term, so splitting pays although the
        CTAs then come in several waves)
      - the larger of the two counts, plus the merge: about 2 us inside a cluster (up to 16 splits, all CTAs
        resident at once: `cluster_slots(n)` says how many CTAs that is for clusters of more than 8), else a merge
        kernel of about 6 us + 0.1 us per split (a launch more in the step's chain; at 9 and 12 requests the count
        that still merges in its clusters beat the next one, which does not, by 2-3.5 us a layer).
      - more CTAs than can be resident come in waves: the full waves stream at the bandwidth, but the CTAs of a
        part-filled last wave run with few others and cannot use what the rest left free - each walks its tiles at a
        lone CTA's pace.  (40-56 requests over 4k keys, one split: 384 CTAs on 296 places took as long as 512;
        three splits took a tenth off the step at 40 and 48 requests, none at 56.)"""
    if _FORCED_SPLITS:
        return max(1, min(_FORCED_SPLITS, tiles))
    key = None
    if cluster_slots is None:
        key = (ctas, tiles, slots, head_dim, total_tiles, ATTN_CLUSTER_MERGE)
        if key in _splits_memo:
            return _splits_memo[key]
        cluster_slots = lambda n: decode_cluster_slots(head_dim, n)
    if total_tiles is None:
        total_tiles = ctas * tiles
    total_tiles = max(min(total_tiles, ctas * tiles), 1)
    tile_us = head_dim / 128.0                              # a lone CTA's time for one tile
    tile_bw_us = 64 * head_dim * 4 / 6.5e6                  # one tile's bytes at the device's bandwidth
    ahead = 3                                               # tiles a CTA requests before it has to wait
    best, best_cost = 1, None
    for n in range(1, max(1, min(64, tiles)) + 1):
        per = -(-tiles // n)                                # the longest request's CTAs
        per_avg = max(total_tiles / (ctas * n), 1.0)
        early = min(total_tiles, min(ctas * n, slots) * ahead)
        t_bw = (total_tiles - early) * tile_bw_us * (1.0 + 2.7 / per_avg)
        t_lat = max(0, per - ahead) * tile_us + 5.0
        if n == 1:
            merge = 0.0
        elif n <= min(MAX_CLUSTER_SPLITS, head_dim) and ATTN_CLUSTER_MERGE and \
                ctas * n <= CLUSTER_FILL * (slots if n <= 8 else min(slots, cluster_slots(n))):
            merge = 2.0
        else:
            merge = 6.0 + 0.1 * n
        t_wave = 0.0
        if ctas * n > slots:
            full, rest = divmod(ctas * n, slots)
            fill_drain = 1.0 + 2.7 / per_avg
            wave = per_avg * max(tile_us, slots * tile_bw_us) * fill_drain
            t_wave = full * wave
            if rest:
                # (the CTAs of a wave end within about a seventh of its length of one another, and the next begin as
                # they do: that much of the last wave runs beside the one before it)
                t_wave += per_avg * max(tile_us, rest * tile_bw_us) * fill_drain - 0.15 * wave
        cost = max(t_bw, t_lat, t_wave) + merge
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = n, cost
    if key is not None:
        if len(_splits_memo) > 4096:
            _splits_memo.clear()
        _splits_memo[key] = best
    return best


_splits_memo: dict = {}
# REINFER_B200_ATTN_SPLITS=n: every decode attention launch splits its keys n ways (a development switch, to measure the model against)
_FORCED_SPLITS = int(os.environ.get("REINFER_B200_ATTN_SPLITS", "0") or 0)


def attention(ctx, q: torch.Tensor, cache: torch.Tensor, group, out: torch.Tensor, QH: int, KH: int, d: int,
              window: int, scale: float) -> None:
    """Attention of a step's tokens over their requests' pages.  float32 (and head sizes the
    tensor-core kernels do not take) runs the plain kernel; bfloat16 runs flash decoding for the
    entries with one token and the paged flash prefill kernel for the others."""
    n_dec, E = ctx.n_decode, ctx.n_entries
    dec_work = pre_work = (0.0, 0.0)
    if _profiler is not None:
        def work(first, last):
            """(flops, bytes) that attention over entries first..last-1 has to do: two products of 2*d per (query head,
            key) pair the causal mask lets through, and every key and value of the request read once."""
            fl = by = 0.0
            for e in range(first, last):
                n, s0 = ctx.q_start[e + 1] - ctx.q_start[e], ctx.start_pos[e]
                pairs = n * s0 + n * (n + 1) / 2
                if window:
                    pairs = min(pairs, n * window)
                fl += 4.0 * QH * d * pairs
                by += ((min(s0 + n, window + n) if window else s0 + n) * KH * 2 + 2 * n * QH) * d * q.element_size()
            return fl, by
        dec_work, pre_work = work(0, n_dec), work(n_dec, E)
    if q.dtype != torch.bfloat16 or d % 8 or d > 256:
        paged_attention_ref(q, cache, group.block_table, ctx.tok_entry, ctx.positions, out, QH, KH, d,
                            group.page_size, window, scale, work=(dec_work[0] + pre_work[0], dec_work[1] + pre_work[1]))
        return
    _need(q.is_contiguous() and out.is_contiguous() and cache.is_contiguous() and group.block_table.is_contiguous(),
          "attention: contiguous")
    gc = fa_group_chunk(QH // KH)
    joined = None
    if n_dec:
        pairs = KH * (QH // KH // gc)
        ctas = n_dec * pairs
        tiles = ctx.decode_kv_tiles[1] if ctx.decode_kv_tiles else -(-ctx.max_kv_len // 64)
        total = ctx.decode_kv_tiles[0] * pairs if ctx.decode_kv_tiles else None
        plan = getattr(ctx, "decode_plan", None)              # a captured step: the split it was made for
        n_splits = max(1, min(int(plan), tiles)) if isinstance(plan, int) and not _FORCED_SPLITS else \
            decode_splits(ctas, tiles, head_dim=d, total_tiles=total)
        decode = fa_decode_tma if (tma_pages(group.page_size) and USE_TMA_ATTENTION) else fa_decode
        if E > n_dec and MIXED_OVERLAP and _profiler is None and not torch.cuda.is_current_stream_capturing():
            # A step with prompt portions beside decoding requests: the two attention kernels read the same inputs
            # and write different rows, and the decoding requests' kernel leaves most SMs idle (a few CTAs with long
            # chains).  It runs on a stream of its own beside the portions' kernel; the main stream goes on when
            # both are done.
            main = torch.cuda.current_stream()
            ready = torch.cuda.Event()
            ready.record(main)
            side = _side_stream(q.device)
            side.wait_event(ready)
            with torch.cuda.stream(side):
                decode(q, cache, group.block_table, ctx.cu_q, ctx.kv_len, out, 0, n_dec, 0, n_splits, QH, KH, d,
                       group.page_size, window, scale, work=dec_work)
                joined = torch.cuda.Event()
                joined.record(side)
        else:
            decode(q, cache, group.block_table, ctx.cu_q, ctx.kv_len, out, 0, n_dec, 0, n_splits, QH, KH, d,
                   group.page_size, window, scale, work=dec_work)
    if E > n_dec and d == 128 and USE_TC_ATTENTION and USE_TMA_ATTENTION and tma_pages(group.page_size):
        fa_prefill_tc(q, cache, group.block_table, ctx.cu_q, ctx.kv_len, out, n_dec, E - n_dec,
                      [ctx.q_start[e + 1] - ctx.q_start[e] for e in range(n_dec, E)], QH, KH, d, group.page_size, window, scale,
                      work=pre_work)
    elif E > n_dec:
        tpt = 64 // gc
        n_tiles = sum(-(-(ctx.q_start[e + 1] - ctx.q_start[e]) // tpt) for e in range(n_dec, E))
        prefill = fa_prefill_tma if (tma_pages(group.page_size) and USE_TMA_ATTENTION) else fa_prefill
        prefill(q, cache, group.block_table, ctx.cu_q, ctx.kv_len, out, n_dec, E - n_dec, n_tiles, QH, KH, d,
                group.page_size, window, scale, work=pre_work)
    if joined is not None:
        torch.cuda.current_stream().wait_event(joined)


def sample(logits: torch.Tensor, row_idx: Optional[torch.Tensor], params: torch.Tensor, history: Optional[torch.Tensor],
           work: torch.Tensor, out_tokens: torch.Tensor, rows: int) -> None:
    """params: uint8 tensor holding `rows` RbSampleParams records (see sampling/sampler.py)."""
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "sample: float32 logits")
    vocab = logits.shape[1]
    hist_cap = history.shape[1] if history is not None else 0
    _need(work.numel() >= rows * vocab and work.dtype == torch.float32, "sample: scratch of rows*vocab floats")
    _check(lib().rb_sample(_p(logits), c_longlong(logits.stride(0)), _p(row_idx), _p(params), _p(history),
                           c_int(hist_cap), _p(work), _p(out_tokens), c_int(rows), c_int(vocab), _stream()), "sample")


def sample_slots(logits: torch.Tensor, row_slot: torch.Tensor, slot_params: torch.Tensor, slot_history: torch.Tensor,
                 slot_token: torch.Tensor, work: torch.Tensor, out_tokens: torch.Tensor, rows: int) -> None:
    """One token per row of `logits`, every request's parameters, seed, draw count and recent tokens taken from
    (and the token written to) its slot: row r belongs to slot row_slot[r] (csrc/sampler.cu)."""
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "sample_slots: float32 logits")
    vocab = logits.shape[1]
    _need(work.numel() >= rows * vocab and work.dtype == torch.float32, "sample_slots: scratch of rows*vocab floats")
    _need(row_slot.dtype == torch.int32 and slot_token.dtype == torch.int32 and slot_history.dtype == torch.int32 and
          slot_params.dtype == torch.uint8 and slot_params.is_contiguous() and slot_history.is_contiguous(),
          "sample_slots: int32 tables, records as bytes")
    _check(lib().rb_sample_slots(_p(logits), c_longlong(logits.stride(0)), _p(row_slot), _p(slot_params), _p(slot_history),
                                 c_int(slot_history.shape[1]), _p(slot_token), _p(work), _p(out_tokens), c_int(rows),
                                 c_int(vocab), _stream()), "sample_slots")


_gemm_ws = None
GEMM_WS_FLOATS = 8 << 20          # 32 MB of split-K partials


def set_gemm_token_lanes(value: int) -> int:
    """Which form the tensor-core product over several token tiles takes: 1 a token per accumulator lane, 0 a
    feature per lane.  Returns the old setting; for tests and comparisons."""
    return int(lib().rb_set_gemm_token_lanes(c_int(int(value))))


def set_gemm_tile_features(value: int) -> int:
    """Weight rows per tile of the products over several token tiles (token-lane forms): 256 (four stages in
    flight), 224 (five), or 0 = chosen per product by the rounds its tiles need over the SMs.  Returns the old
    setting; for tests and comparisons."""
    return int(lib().rb_set_gemm_tile_features(c_int(int(value))))


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, accumulate: bool = False, splits: int = 0,
              row_scale=None) -> None:
    """c[T,N] (=|+=) a[T,K] @ w[N,K]^T on the tensor cores (tcgen05, TMA); bf16 operands, float
    accumulation, c bfloat16 or float32.  Operands that TMA cannot address (a row stride that is no
    multiple of 8 elements, a base that is not 16-byte aligned) go to the plain kernel instead."""
    global _gemm_ws
    T, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and tuple(c.shape) == (T, N), "gemm: shapes")
    _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_bf16: bfloat16 operands")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1, "gemm: rows contiguous")
    if a.stride(0) % 8 or w.stride(0) % 8 or a.data_ptr() % 16 or w.data_ptr() % 16:
        _need(row_scale is None, "gemm: row factors need operands that TMA can address")
        return gemm_ref(a, w, c, accumulate)
    if _gemm_ws is None or _gemm_ws.device != a.device:
        _gemm_ws = torch.empty(GEMM_WS_FLOATS, dtype=torch.float32, device=a.device)
    nw, nb = _next_range(w) if T <= STREAMING_TOKENS else (c_void_p(0), c_longlong(0))
    _check(lib().rb_gemm_bf16(_p(a), _p(w), _p(c), c_int(dt(c)), c_int(int(accumulate)), c_int(T), c_int(N), c_int(K),
                              c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(c.stride(0)),
                              _p(_gemm_ws), c_longlong(_gemm_ws.numel()), c_int(splits), nw, nb,
                              *_row_scale_args(row_scale, T), _stream()), f"gemm {N}x{K}",
           2.0 * T * N * K, 2.0 * (T * K + N * K) + T * N * c.element_size())


# REINFER_B200_QKV_HEADS=0: the q/k/v projection and the per-head work as two kernels at every size (a development switch).
QKV_HEADS = os.environ.get("REINFER_B200_QKV_HEADS", "1") != "0"


def gemm_qkv_heads(a: torch.Tensor, w_qkv: torch.Tensor, q_out: torch.Tensor, cache: torch.Tensor, kv_slot: torch.Tensor,
                   cs_table: torch.Tensor, q_w: torch.Tensor, k_w: torch.Tensor, QH: int, KH: int, page_size: int, eps: float,
                   row_scale=None) -> bool:
    """The q/k/v projection of a prompt portion with the per-head work in its epilogue (heads of 128): q_out [T, QH, 128]
    gets the normalised, rotated queries, the cache pages the keys and values at kv_slot.  cs_table [T, 64, 2] float32
    from rope_table.  Returns False (and does nothing) where this form does not apply - at most 256 tokens, operands
    that TMA cannot address - and the caller runs the product and qknorm_rope_append one after the other."""
    T, K = a.shape
    if not QKV_HEADS:
        return False
    if T <= 256 or a.dtype != torch.bfloat16 or w_qkv.dtype != torch.bfloat16 or q_out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        return False
    if row_scale is not None and not row_scale_ok(T):
        return False
    if a.stride(1) != 1 or w_qkv.stride(1) != 1 or a.stride(0) % 8 or w_qkv.stride(0) % 8 or a.data_ptr() % 16 or w_qkv.data_ptr() % 16:
        return False
    _need(w_qkv.shape == ((QH + 2 * KH) * 128, K), "gemm_qkv_heads: weight shape")
    _need(q_out.is_contiguous() and tuple(q_out.shape) == (T, QH, 128) and cache.is_contiguous(), "gemm_qkv_heads: q_out [T, QH, 128], cache contiguous")
    _need(q_w.dtype == k_w.dtype and q_w.numel() == 128 and k_w.numel() == 128 and q_w.is_contiguous() and k_w.is_contiguous(),
          "gemm_qkv_heads: norm weights [128] of one dtype")
    _need(cs_table.dtype == torch.float32 and cs_table.is_contiguous() and cs_table.numel() == T * 128, "gemm_qkv_heads: table [T, 64, 2] float32")
    _need(kv_slot.dtype == torch.int32 and kv_slot.numel() >= T, "gemm_qkv_heads: kv_slot int32 [T]")
    N = (QH + 2 * KH) * 128
    _check(lib().rb_gemm_qkv_heads(_p(a), _p(w_qkv), c_int(T), c_int(K), c_longlong(a.stride(0)), c_longlong(w_qkv.stride(0)),
                                   c_int(QH), c_int(KH), _p(q_out), _p(cache), _p(kv_slot), _p(cs_table), _p(q_w), _p(k_w),
                                   c_int(dt(q_w)), c_float(eps), c_int(page_size), *_row_scale_args(row_scale, T), _stream()),
           f"gemm+heads {N}x{K}", 2.0 * T * N * K, float(T * K * 2 + N * K * 2 + T * N * 2))
    return True


def gemm_qkv_heads_stream(a, w_qkv: torch.Tensor, q_out: torch.Tensor, cache: torch.Tensor, kv_slot: Optional[torch.Tensor],
                          positions: torch.Tensor, inv_freq: torch.Tensor, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor],
                          QH: int, KH: int, page_size: int, eps: float, row_scale=None) -> bool:
    """The q/k/v projection of a decode step's few rows (heads of 128) whose cluster does the per-head work on its sums:
    q_out [T, QH, 128] gets the normalised, rotated queries, the cache pages the keys and values at kv_slot (None:
    nothing is stored).  Returns False (and does nothing) where this form does not apply, and the caller runs the
    product and qknorm_rope_append one after the other."""
    T, K = a.shape
    if not (QKV_HEADS and 0 < T <= STREAMING_TOKENS and K >= 128 and a.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16 and
            q_out.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16):
        return False
    if a.stride(1) != 1 or w_qkv.stride(1) != 1 or a.stride(0) % 8 or w_qkv.stride(0) % 8 or a.data_ptr() % 16 or w_qkv.data_ptr() % 16:
        return False
    _need(w_qkv.shape == ((QH + 2 * KH) * 128, K), "gemm_qkv_heads_stream: weight shape")
    _need(q_out.is_contiguous() and tuple(q_out.shape) == (T, QH, 128) and cache.is_contiguous(), "gemm_qkv_heads_stream: q_out [T, QH, 128], cache contiguous")
    _need((q_w is None) == (k_w is None), "gemm_qkv_heads_stream: q and k norm weights come together")
    if q_w is not None:
        _need(q_w.dtype == k_w.dtype and q_w.numel() == 128 and k_w.numel() == 128 and q_w.is_contiguous() and k_w.is_contiguous(),
              "gemm_qkv_heads_stream: norm weights [128] of one dtype")
    _need(inv_freq.dtype == torch.float32 and inv_freq.numel() == 64 and inv_freq.is_contiguous(), "gemm_qkv_heads_stream: inv_freq float32 [64]")
    _need(positions.dtype == torch.int32 and positions.numel() >= T, "gemm_qkv_heads_stream: positions int32 [T]")
    _need(kv_slot is None or (kv_slot.dtype == torch.int32 and kv_slot.numel() >= T), "gemm_qkv_heads_stream: kv_slot int32 [T]")
    N = (QH + 2 * KH) * 128
    nw, nb = _next_range(w_qkv)
    _check(lib().rb_gemm_qkv_heads_stream(_p(a), _p(w_qkv), c_int(T), c_int(K), c_longlong(a.stride(0)), c_longlong(w_qkv.stride(0)),
                                          c_int(QH), c_int(KH), _p(q_out), _p(cache), _p(kv_slot), _p(positions), _p(inv_freq),
                                          _p(q_w), _p(k_w), c_int(dt(q_w) if q_w is not None else 0), c_float(eps), c_int(page_size),
                                          nw, nb, *_row_scale_args(row_scale, T), _stream()),
           f"gemm+heads {N}x{K}", 2.0 * T * N * K, float(T * K * 2 + N * K * 2 + T * N * 2))
    return True


def gemm_bf16_partials(a: torch.Tensor, w: torch.Tensor, row_scale=None) -> Optional[torch.Tensor]:
    """Partial sums [S, T, N] (float32) of a[T,K] @ w[N,K]^T over S ranges of K, for a consumer that adds them
    up itself (add_rmsnorm with a stacked delta): the split product then needs no reduction of its own, and
    none of its CTAs waits for another.  None if this product is not one for the streaming kernel (more than
    STREAMING_TOKENS tokens, operands that TMA cannot address): the caller then runs the plain form."""
    T, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K, "gemm: shapes")
    if not (0 < T <= STREAMING_TOKENS and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
        return None
    if a.stride(1) != 1 or w.stride(1) != 1 or a.stride(0) % 8 or w.stride(0) % 8 or a.data_ptr() % 16 or w.data_ptr() % 16:
        return None
    S = int(lib().rb_gemm_partials_plan(c_int(T), c_int(N), c_int(K)))
    out = torch.empty((S, T, N), dtype=torch.float32, device=a.device)
    nw, nb = _next_range(w)
    _check(lib().rb_gemm_bf16_partials(_p(a), _p(w), _p(out), c_int(S), c_int(T), c_int(N), c_int(K),
                                       c_longlong(a.stride(0)), c_longlong(w.stride(0)), nw, nb,
                                       *_row_scale_args(row_scale, T), _stream()), f"gemm {N}x{K}",
           2.0 * T * N * K, 2.0 * (T * K + N * K) + 4.0 * S * T * N)
    return out


# REINFER_B200_PRODUCT_NORM=0: a decode step's o and down projections never prepare the next norm's rows themselves
# (they leave partial sums, or add into the residual, and the norm runs as a kernel of its own).
PRODUCT_NORM = os.environ.get("REINFER_B200_PRODUCT_NORM", "1") != "0"


def gemm_bf16_residual_norm(a: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, norm_w: torch.Tensor, row_scale=None):
    """residual[T,N] (float32) += a[T,K] @ w[N,K]^T for a decode step's few rows, the product reduced inside a
    cluster whose CTAs also prepare what the RMS norm with weight norm_w would make of the new residual: returns
    (rows, sumsq) as residual_rowscale does (rows = bfloat16(residual * norm_w), sumsq [T, N/128] the sum of squares
    by tiles of 128 columns), or None (and does nothing) where this form does not apply."""
    T, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and tuple(residual.shape) == (T, N), "gemm: shapes")
    if not (PRODUCT_NORM and 0 < T <= STREAMING_TOKENS and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and
            residual.dtype == torch.float32 and N % 128 == 0 and K >= 128 and norm_w.numel() == N and norm_w.is_contiguous() and
            norm_w.dtype in (torch.float32, torch.bfloat16) and norm_w.data_ptr() % 16 == 0):
        return None
    if a.stride(1) != 1 or w.stride(1) != 1 or a.stride(0) % 8 or w.stride(0) % 8 or a.data_ptr() % 16 or w.data_ptr() % 16 or \
            residual.stride(1) != 1 or residual.stride(0) % 4 or residual.data_ptr() % 16:
        return None
    rows = torch.empty((T, N), dtype=torch.bfloat16, device=a.device)
    sumsq = torch.empty((T, N // 128), dtype=torch.float32, device=a.device)
    nw, nb = _next_range(w)
    _check(lib().rb_gemm_bf16_residual_norm(_p(a), _p(w), _p(residual), c_int(T), c_int(N), c_int(K), c_longlong(a.stride(0)),
                                            c_longlong(w.stride(0)), c_longlong(residual.stride(0)), _p(norm_w), c_int(dt(norm_w)),
                                            _p(rows), _p(sumsq), nw, nb, *_row_scale_args(row_scale, T), _stream()),
           f"gemm+norm {N}x{K}", 2.0 * T * N * K, 2.0 * (T * K + N * K) + 14.0 * T * N)
    return rows, sumsq


def gemm_bf16_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, splits: int = 0, row_scale=None) -> bool:
    """out[T,F] (bf16) = silu(a Wg^T) * (a Wu^T), w_gate_up = [Wg; Wu] of shape [2F, K]: one tensor-core
    product with two accumulators and the activation in its epilogue.  Returns False (and does
    nothing) if TMA cannot address the operands; the caller then runs the two-kernel form."""
    T, K = a.shape
    F_ = out.shape[1]
    _need(w_gate_up.shape == (2 * F_, K) and out.shape[0] == T, "gemm_swiglu: shapes")
    _need(a.dtype == w_gate_up.dtype == out.dtype == torch.bfloat16, "gemm_swiglu: bfloat16 tensors")
    _need(a.stride(1) == 1 and w_gate_up.stride(1) == 1 and out.stride(1) == 1, "gemm_swiglu: rows contiguous")
    if a.stride(0) % 8 or w_gate_up.stride(0) % 8 or a.data_ptr() % 16 or w_gate_up.data_ptr() % 16:
        return False
    nw, nb = _next_range(w_gate_up) if T <= STREAMING_TOKENS else (c_void_p(0), c_longlong(0))
    _check(lib().rb_gemm_bf16_swiglu(_p(a), _p(w_gate_up), _p(out), c_int(T), c_int(F_), c_int(K),
                                     c_longlong(a.stride(0)), c_longlong(w_gate_up.stride(0)), c_longlong(out.stride(0)),
                                     c_int(splits), nw, nb, *_row_scale_args(row_scale, T), _stream()),
           f"gemm+swiglu {2 * F_}x{K}", 4.0 * T * F_ * K, 2.0 * (T * K + 2 * F_ * K + T * F_))
    return True


def random_normal(out: torch.Tensor, base: int, mean: float, std: float) -> None:
    """out[i] = mean + std * n_i, n_i the i-th normal of the counter stream that starts at `base`
    (weights/random.py states the function); out float32 or bfloat16, contiguous."""
    _need(out.is_contiguous(), "random_normal: contiguous tensor")
    _check(lib().rb_random_normal(_p(out), c_int(dt(out)), c_longlong(out.numel()), ctypes.c_ulonglong(base & ((1 << 64) - 1)),
                                  ctypes.c_double(mean), ctypes.c_double(std), _stream()), "random_normal")


def random_ints(out: torch.Tensor, base: int) -> None:
    _need(out.is_contiguous() and out.dtype == torch.int32, "random_ints: contiguous int32 tensor")
    _check(lib().rb_random_ints(_p(out), c_longlong(out.numel()), ctypes.c_ulonglong(base & ((1 << 64) - 1)), _stream()),
           "random_ints")


def kernel_error(reset: bool = True) -> int:
    """The error word that a kernel sets when one of its bounded waits gives up (0 = none).
    Synchronises the device."""
    words = [int(fn(c_int(int(reset)))) for fn in (lib().rb_gemm_error, lib().rb_attn_error, lib().rb_attn_tc_error,
                                                   lib().rb_selftest_error)]
    if reset and any(words):
        lib().rb_status_clear()
    return next((w for w in words if w), 0)


_status_word = None
STATUS_UNITS = {1: "tensor-core product (gemm_tc.cu)", 2: "paged attention (attention_tma.cu)",
                3: "tensor-core prefill attention (attention_tc.cu)", 4: "bounded-wait self-test (selftest.cu)"}


def status_word() -> int:
    """The host's copy of the kernels' error word: 0, or the code of the first bounded wait that gave up.
    A plain load from pinned memory that the kernels write to; no call into the device, no synchronisation.
    What it shows is complete for every kernel the host has already waited for."""
    global _status_word
    if _status_word is None:
        fn = lib().rb_status_host
        fn.restype = ctypes.POINTER(c_int)
        ptr = fn()
        if not ptr:
            raise KernelError(f"status word: {lib().rb_last_error().decode()}")
        _status_word = ptr
    return int(_status_word[0])


def describe_status(code: int) -> str:
    unit, where = (code >> 16) & 0xFF, code & 0xFF
    return f"a bounded wait gave up at point {where} of the {STATUS_UNITS.get(unit, f'unit {unit}')}"


def clear_status() -> int:
    """Clear the status word and the kernels' own words after an error was handled (synchronises the device)."""
    status_word()
    return int(lib().rb_status_clear())


def test_bounded_wait(limit_ns: int, gave_up: Optional[torch.Tensor] = None) -> None:
    """Launch the self-test kernel whose wait nobody answers (selftest.cu); it gives up after `limit_ns`."""
    status_word()                       # the word must be bound before a kernel can write it
    _check(lib().rb_test_bounded_wait(ctypes.c_ulonglong(int(limit_ns)), _p(gave_up), _stream()), "test_bounded_wait")


def sample_params_size() -> int:
    return int(lib().rb_sample_params_size())
