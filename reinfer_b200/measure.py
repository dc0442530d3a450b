"""Measurements on random-weight models of given shapes: what `bench.py` prints and what
`python -m reinfer_b200 bench` shows.  A shape is a config.json: one of the files under
`reinfer_b200/shapes/` (qwen3-8b, qwen3-4b, qwen3-32b: the three sizes the measurements are
quoted on) or any path.  The model is built through the registry like every other, with
weights drawn on the device by the seeded generator, and driven through the public entry
points: `Engine.step` for the prefill, `LLM.step` for decoding and for the mixed run.

The reference measures through `run --perf` (bin/reinfer/src/main.rs:700-727) and an HTTP
load generator (bench/gate-fixture.md:24-28, bench/notes.md:1534: concurrent requests);
here seeded uniform-random token ids of the stated lengths stand in for any data set.

  prefill(T)            one request of T tokens in one step; tokens/s and the fraction of the
                        tensor-core peak (flops of the products and of causal attention / time)
  decode(B, ...)        B requests at a given context decode together; per step: the device's
                        time (the captured step - every layer, the head, the sampler - replayed
                        back to back) and the time through `LLM.step` (scheduler, tables from
                        pinned memory, graph, sampler, ids back to pinned memory)
  mixed(n, lo, hi, ...) n requests with prompt lengths uniform in [lo, hi] arrive at once; prompts
                        are cut under the token budget and run beside the others' decode tokens
  segments(...)         one step launched eagerly with an event behind every launch: time, achieved
                        TFLOP/s and GB/s by kernel family
"""
from __future__ import annotations

import json
import os
import time
from typing import Dict, List, Optional

SHAPES_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "shapes")


def shape_path(name: str) -> str:
    """A shape's config.json: a path, or the name of a file under reinfer_b200/shapes (with or without the family's
    prefix: '8b' = 'qwen3-8b')."""
    if os.path.isfile(name):
        return name
    if os.path.isfile(os.path.join(name, "config.json")):
        return os.path.join(name, "config.json")
    known = sorted(f[:-5] for f in os.listdir(SHAPES_DIR) if f.endswith(".json"))
    for cand in known:
        if name.lower() == cand or cand.endswith("-" + name.lower()):
            return os.path.join(SHAPES_DIR, cand + ".json")
    raise FileNotFoundError(f"shape {name!r}: not a config.json and not one of {known}")


def load_shape(name: str, layers: Optional[int] = None):
    """(raw config, typed config, layers of the full model).  `layers` builds fewer layers of the same sizes."""
    from .config.registry import resolve_architecture
    with open(shape_path(name)) as f:
        raw = json.load(f)
    full = int(raw.get("num_hidden_layers", 0))
    if layers:
        raw["num_hidden_layers"] = int(layers)
    arch = resolve_architecture(raw)
    return raw, arch.config_cls.from_dict(raw), full


def peaks(root: Optional[str] = None):
    """(copy GB/s, bf16 TFLOP/s burst, sustained, 'measured'|'fallback') from MEASURED_PEAKS.json beside the package."""
    root = root or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, 1590.0, 1400.0, "fallback"


class Bench:
    """One engine of one shape, and the runs on it."""

    def __init__(self, shape: str, layers: Optional[int] = None, page_size: int = 16, dtype: str = "bfloat16",
                 pool_tokens: int = 0, max_num_seqs: int = 65, seed: int = 0, memory_fraction: float = 0.9):
        import torch
        from .engine import Engine
        self.torch = torch
        self.raw, self.cfg, self.full_layers = load_shape(shape, layers)
        self.layers = int(self.raw["num_hidden_layers"])
        t0 = time.time()
        kw = dict(max_tokens=pool_tokens) if pool_tokens else dict(memory_fraction=memory_fraction)
        self.engine = Engine.from_config(self.cfg, seed=seed, dtype=dtype, page_size=page_size,
                                         max_num_seqs=max_num_seqs, **kw)
        torch.cuda.synchronize()
        self.load_s = time.time() - t0
        self.page_size = page_size
        self.vocab = self.engine.vocab_size
        self.gen = torch.Generator().manual_seed(seed)
        self._account()

    # ---- what a step has to move and to compute ------------------------------------------------------
    def _account(self) -> None:
        """Bytes of the weights that a step reads once (every tensor but a gathered embedding table), bytes of cache
        per token, and the multiply-adds per token of the products."""
        model = self.engine.model
        spec = model.spec
        isz = 2 if self.engine.dtype == self.torch.bfloat16 else 4
        tied = bool(getattr(model.lm_head, "tied", False))
        total = mat = 0
        for name, ps in model.param_specs().items():
            n = 1
            for s in ps.shape:
                n *= s
            if name == spec.embedding.prefix + "weight":
                if tied:
                    total += n                              # read as the output matrix
                continue
            if name.startswith(spec.lm_head.prefix) and ps.optional and tied:
                continue
            total += n
            if len(ps.shape) == 2 and not name.startswith(spec.lm_head.prefix):
                mat += n
        self.weight_bytes = total * isz
        self.matmul_params = mat                            # without the output matrix (it runs on wanted rows only)
        self.head_params = spec.vocab_size * spec.hidden_size
        paged, _ = model.cache_layout()
        self.kv_bytes_per_token = sum(2 * s.kv_heads * s.head_dim * isz for s in paged.values())
        self.attn_dims = [(l.mixer.QH, l.mixer.d) for i, _ in model.run for l in [model.layers[i]]
                          if l.mixer is not None and hasattr(l.mixer, "QH")]

    def prefill_flops(self, T: int, rows: int = 1) -> float:
        attn = sum(4.0 * qh * d * T * (T + 1) / 2 for qh, d in self.attn_dims)     # QK^T and PV over the causal half
        return 2.0 * T * self.matmul_params + attn + 2.0 * rows * self.head_params

    def tokens(self, n: int) -> List[int]:
        return self.torch.randint(0, self.vocab, (n,), generator=self.gen).tolist()

    def _ev(self):
        return self.torch.cuda.Event(enable_timing=True)

    # ---- prefill -------------------------------------------------------------------------------------
    def prefill(self, T: int = 2048, repeats: int = 3) -> Dict:
        from .engine import StepEntry
        torch, ms = self.torch, []
        for it in range(repeats):
            toks = self.tokens(T)
            e0, e1 = self._ev(), self._ev()
            torch.cuda.synchronize()
            e0.record()
            self.engine.step([StepEntry("prefill", toks, [T - 1])])
            e1.record()
            torch.cuda.synchronize()
            ms.append(e0.elapsed_time(e1))
            self.engine.finish("prefill")
        best = min(ms[1:]) if len(ms) > 1 else ms[0]
        return {"tokens": T, "ms": best, "value": T / best * 1e3, "flops": self.prefill_flops(T)}

    # ---- decode --------------------------------------------------------------------------------------
    def decode(self, B: int, steps: int, warmup: int, context: int) -> Dict:
        """Fill B requests so that they are at about `context` tokens when the timed steps end; time `steps` steps
        through `LLM.step` by the wall clock, then the same step's graph alone by CUDA events."""
        from .engine.llm import LLM
        from .sampling import SamplingParams
        torch, engine = self.torch, self.engine
        # the request admitted first decodes while the others still run their prompts (a prompt takes context / 2,048
        # steps): leave that many tokens of room, so that no request passes `context` (and no block table outgrows the
        # captured step's width) before the timed steps end
        start_len = max(context - steps - warmup - B * (-(-context // 2048) + 1) - 2, 1)
        llm = LLM(engine=engine, max_batch_tokens=2048, seed=0)
        sp = SamplingParams(temperature=0.0, max_tokens=1 << 20, ignore_eos=True)
        for _ in range(B):
            llm.add_request(self.tokens(start_len), sp)
        while any(r.in_prefill for r in llm.scheduler.running) or llm.scheduler.waiting:
            llm.step()
        for _ in range(warmup):
            llm.step()
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        for _ in range(steps):
            llm.step()
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - w0) / steps * 1e3
        if len(llm.scheduler.running) != B or llm.scheduler.waiting:
            raise RuntimeError("decode run: a request left the batch during the timed steps")
        kv_tokens = sum(engine.cache.length(r.request_id) for r in llm.scheduler.running)
        bucket = B if B <= 8 else -(-B // 8) * 8
        graph = max((g for key, g in engine._graphs.items() if key[0] == bucket), key=lambda g: g.meta.numel())
        for _ in range(3):
            graph.graph.replay()
        torch.cuda.synchronize()
        e0, e1 = self._ev(), self._ev()
        e0.record()
        for _ in range(steps):
            graph.graph.replay()
        e1.record()
        torch.cuda.synchronize()
        dev_ms = e0.elapsed_time(e1) / steps
        out = {"batch": B, "context": context, "ms_device": dev_ms, "ms_e2e": wall_ms, "launches_per_step": graph.n_launches,
               "kv_tokens": kv_tokens, "bytes": self.weight_bytes + kv_tokens * self.kv_bytes_per_token,
               "h2d_bytes_per_step": int(graph.meta.numel()) * 4, "d2h_bytes_per_step": B * 4,
               "steps_launched_ahead": llm.steps_launched_ahead}
        for r in list(llm.scheduler.running):
            llm.abort(r.request_id)
        while llm.has_work():
            llm.step()                                    # a step launched ahead is read and dropped
        return out

    # ---- many requests at once ----------------------------------------------------------------------------
    def mixed(self, n_requests: int = 32, lo: int = 128, hi: int = 4096, budget: int = 2048, new_tokens: int = 128,
              seed: int = 0, passes: int = 2) -> Dict:
        """`n_requests` arrive together with prompt lengths uniform in [lo, hi]; every one generates `new_tokens`.
        The same requests run `passes` times through one entry point and the last pass is the one reported: the
        passes before it pay for what a serving process pays once (first launches, the captures of the decode
        steps' graphs, which belong to the entry point's sampler and go with it)."""
        from .engine.llm import LLM
        from .sampling import SamplingParams
        torch = self.torch
        g = torch.Generator().manual_seed(seed)
        lengths = torch.randint(lo, hi + 1, (n_requests,), generator=g).tolist()
        prompts = [self.tokens(n) for n in lengths]
        llm = LLM(engine=self.engine, max_batch_tokens=budget, seed=seed)
        sp = SamplingParams(temperature=0.0, max_tokens=new_tokens, ignore_eos=True)
        for _ in range(max(1, passes)):
            ids = [llm.add_request(p, sp) for p in prompts]
            ahead0, pre0 = llm.steps_launched_ahead, llm.scheduler.stats["preemptions"]
            first: Dict = {}
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            steps = 0
            while llm.has_work():
                llm.step()
                steps += 1
                now = time.perf_counter() - t0
                for rid in ids:
                    if rid not in first and llm.requests[rid].output:
                        first[rid] = now
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            gen = sum(len(llm.requests.pop(rid).output) for rid in ids)
        ttft = sorted(first.values())
        return {"requests": n_requests, "prompt_tokens": sum(lengths), "generated_tokens": gen, "seconds": dt, "steps": steps,
                "tokens_per_s": (sum(lengths) + gen) / dt, "generated_per_s": gen / dt, "budget": budget,
                "preemptions": llm.scheduler.stats["preemptions"] - pre0, "ttft_p50_s": ttft[len(ttft) // 2] if ttft else None,
                "ttft_max_s": ttft[-1] if ttft else None, "steps_launched_ahead": llm.steps_launched_ahead - ahead0,
                "passes": max(1, passes)}

    # ---- where a step's time goes ----------------------------------------------------------------------------
    def segments(self, kind: str, B: int = 8, context: int = 4096, T: int = 2048) -> Dict:
        """One step of the kind ('decode': B requests at `context`; 'prefill': T tokens), launched eagerly with an
        event behind every launch (ops.SegmentProfiler).  -> name -> {n, us, tflops, gbs}."""
        from . import ops
        from .engine import StepEntry
        torch, engine = self.torch, self.engine
        graphs, engine.cuda_graphs = engine.cuda_graphs, False
        prof = ops.SegmentProfiler()
        try:
            if kind == "decode":
                for b in range(B):
                    toks = self.tokens(context - 2)
                    for i in range(0, len(toks), 2048):
                        engine.step([StepEntry(("seg", b), toks[i:i + 2048], [])])
                entries = [StepEntry(("seg", b), [5 + b], [0]) for b in range(B)]
                engine.step(entries)                                    # warm
                entries = [StepEntry(("seg", b), [7 + b], [0]) for b in range(B)]
            else:
                engine.step([StepEntry(("seg", "w"), self.tokens(T), [T - 1])])
                engine.finish(("seg", "w"))
                entries = [StepEntry(("seg", 0), self.tokens(T), [T - 1])]
            torch.cuda.synchronize()
            # the host needs a few milliseconds to queue a step's launches and events: the device sleeps meanwhile, so
            # that no launch waits for the host and a launch's span is the kernel's own time
            torch.cuda._sleep(60_000_000 if kind == "decode" else 20_000_000)
            old = ops.set_profiler(prof)
            prof.begin()
            try:
                engine.step(entries)
            finally:
                ops.set_profiler(old)
            out = prof.summary()
        finally:
            engine.cuda_graphs = graphs
            for rid in list(engine.cache.live()):
                if isinstance(rid, tuple) and rid and rid[0] == "seg":
                    engine.finish(rid)
        return out


def segment_table(seg: Dict, hbm_gbs: float, tflops: float) -> List[str]:
    """Lines of a table: family, launches, microseconds, share, achieved rate and its fraction of the peak."""
    total = sum(d["us"] for d in seg.values()) or 1.0
    lines = [f"{'segment':28s} {'n':>4s} {'us':>9s} {'share':>6s} {'TFLOP/s':>8s} {'GB/s':>8s} {'of peak':>8s}"]
    for name, d in sorted(seg.items(), key=lambda kv: -kv[1]["us"]):
        frac = max(d["tflops"] / tflops, d["gbs"] / hbm_gbs)
        lines.append(f"{name:28s} {d['n']:4d} {d['us']:9.1f} {100 * d['us'] / total:5.1f}% {d['tflops']:8.1f} {d['gbs']:8.0f} {100 * frac:7.1f}%")
    lines.append(f"{'total':28s} {sum(d['n'] for d in seg.values()):4d} {total:9.1f}")
    return lines


def compact_segments(seg: Dict, top: int = 6) -> Dict:
    """The `top` segments by time as {name: [us, TFLOP/s, GB/s]} for a one-line record."""
    keep = sorted(seg.items(), key=lambda kv: -kv[1]["us"])[:top]
    return {k: [round(d["us"], 1), round(d["tflops"], 1), round(d["gbs"])] for k, d in keep}
