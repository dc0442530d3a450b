"""The Python entry point: `LLM(model_dir).generate(prompt_token_ids, SamplingParams)`.
It joins the scheduler, the engine's step function and the GPU sampler in the loop that
the reference runs in bin/reinfer/src/sched_loop.rs:564-587, 691-695 (admit and schedule,
step, sample, finish), with prompts' portions and decoded tokens in ONE step call instead
of separate engine calls.  Token ids in, token ids out: the tokenizer is not part of this
engine.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..config.registry import resolve_eos
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, request_seed
from .admission import AdmissionLimits, EstimateAdmission
from .engine import Engine, EngineError, StepEntry
from .scheduler import RUNNING, Request, Scheduler


@dataclass
class RequestOutput:
    request_id: Hashable
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: Optional[str]
    preemptions: int = 0


class LLM:
    def __init__(self, model: Optional[str] = None, *, engine: Optional[Engine] = None, dtype="bfloat16",
                 max_num_seqs: int = 64, max_batch_tokens: int = 2048, max_chunk: Optional[int] = None,
                 page_size: int = 64, num_pages: Optional[int] = None, max_model_len: Optional[int] = None,
                 seed: int = 0, device="cuda:0", memory_fraction: float = 0.9, admission: str = "pages"):
        """admission: "pages" admits a request when the free pages cover its prompt; "estimate" asks in addition
        for the estimated peak of everything running to fit the pool (engine/admission.py)."""
        if admission not in ("pages", "estimate"):
            raise ValueError(f"admission {admission!r}: pages or estimate")
        if engine is None:
            if model is None:
                raise ValueError("LLM needs a model folder or an engine")
            engine = Engine.from_model_dir(model, dtype=dtype, device=device, page_size=page_size,
                                           num_pages=num_pages, max_num_seqs=max_num_seqs,
                                           memory_fraction=memory_fraction)
        self.engine = engine
        self.seed = int(seed)
        cfg = engine.config
        self.max_model_len = int(max_model_len or getattr(cfg, "max_position_embeddings", 0) or 0) or None
        self.eos = resolve_eos(cfg, model)
        batch_tokens = max(max_batch_tokens, engine.cache.max_seqs)
        estimate = None
        if admission == "estimate":
            estimate = EstimateAdmission(AdmissionLimits(pool_tokens=engine.cache.total_pages() * engine.cache.page_size,
                                                         max_requests=engine.cache.max_seqs, max_batch_tokens=batch_tokens))
        self.scheduler = Scheduler(engine.cache, max_batch_tokens=batch_tokens,
                                   max_chunk=max_chunk, eos_token_ids=self.eos, max_model_len=self.max_model_len,
                                   release=engine.finish, admission=estimate)
        self.sampler = Sampler(engine.vocab_size, -(-engine.cache.max_seqs // 8) * 8, engine.device, storage=engine.storage)
        engine.on_admit = self._admitted            # a request's slot gets its sampler record
        engine.epilogue = self.sampler.launch_slots  # the sampler runs right behind the forward pass, on the device's tables
        self._next_id = 0
        self.requests: Dict[Hashable, Request] = {}
        self.last_stats: Dict[str, float] = {}
        # REINFER_B200_STEP_PROFILE=decode|prefill[:every]: every so many steps (20) of that kind run eagerly with an
        # event behind every launch; `profile_report()` (the command line prints it at the end) gives their mean by
        # kernel family (the reference's REINFER_DECODE_PROFILE / REINFER_PREFILL_PROFILE, crates/cuda/src/engine.rs:928-1408)
        spec = os.environ.get("REINFER_B200_STEP_PROFILE", "")
        self._profile_kind, _, every = spec.partition(":")
        self._profile_every = max(1, int(every)) if every.isdigit() else 20
        self._profile_seen = 0
        self._profile_runs: List[Dict] = []
        self._launched = None                   # a step launched ahead of its scheduling: (batch, tokens on their way)
        self.steps_launched_ahead = 0           # steps that were launched before the step before them was read
        self.ahead_rows_dropped = 0             # rows of such steps that belonged to requests which had ended

    # ---- requests -----------------------------------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[Hashable] = None) -> Hashable:
        params = params or SamplingParams()
        rid = request_id if request_id is not None else self._next_id
        self._next_id += 1
        for t in prompt_token_ids:
            if not 0 <= int(t) < self.engine.vocab_size:
                raise ValueError(f"token id {t} outside the vocabulary of {self.engine.vocab_size}")
        r = Request(rid, [int(t) for t in prompt_token_ids], params)
        self.scheduler.add(r)
        r.seed = params.seed if params.seed is not None else request_seed(self.seed, r.arrival)
        self.requests[rid] = r
        return rid

    def abort(self, request_id) -> None:
        self.scheduler.abort(request_id)

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._launched is not None

    def _admitted(self, request_id, slot: int) -> None:
        r = self.requests.get(request_id)
        if r is not None:
            self.sampler.assign(slot, r.params, r.seed, r.output)

    # ---- one step -------------------------------------------------------------------------
    def step(self) -> List[Request]:
        """One scheduler decision, one engine step with the sampler behind it, and the reading of its tokens.
        Returns the requests that finished in it.

        The device never waits for the host between two decode steps: as soon as a step is launched and it is
        sure that the same requests decode again after it (nobody waits, nobody reaches its token limit), the
        step after it is launched too - its token ids are not known on the host yet, the embedding takes them
        from the requests' slots on the device, where the sampler has put them.  Only then are the first
        step's tokens read.  A request that turns out to end there (a stop token, end of sequence) has one row
        in the step already running; that row is dropped, its request's pages are given back as always."""
        finished: List[Request] = []
        cur, self._launched = self._launched, None
        if cur is None:
            out = self.scheduler.schedule()
            finished += out.finished
            if not out.batch:
                return finished
            cur = (out.batch, None, None)
        batch, tokens, rows = cur
        ahead = None
        try:
            if tokens is None:
                tokens = self._launch(batch)
            sampling = [s.request for s in batch if s.sample]
            if rows is None:
                rows = list(range(len(sampling)))
            ahead = self._launch_ahead(batch)
            sampled: Dict[Hashable, int] = {}
            if sampling:
                got = tokens.result()
                sampled = {r.request_id: got[k] for r, k in zip(sampling, rows)}
            self.engine.check_status()                  # the tokens have arrived: the step's kernels are over
        except EngineError:
            # a kernel gave up (or the engine refused the step): the requests of this step end with "error" and
            # give back their pages; the engine refuses further steps until `engine.clear_status()`
            for s in batch:
                self.scheduler.fail(s.request)
            raise
        finished += self.scheduler.update(batch, sampled)
        if ahead is not None:
            ahead_requests, ahead_tokens = ahead
            alive = [(k, r) for k, r in enumerate(ahead_requests) if r.state == RUNNING]
            self.ahead_rows_dropped += len(ahead_requests) - len(alive)
            if alive:
                self._launched = (self.scheduler.schedule_decode([r for _, r in alive]), ahead_tokens, [k for k, _ in alive])
        return finished

    def _launch(self, batch):
        """Run the batch through the engine (the sampler is its epilogue) and start the tokens' way to the host."""
        entries = [StepEntry(s.request.request_id, s.tokens, [len(s.tokens) - 1] if s.sample else []) for s in batch]
        if self._profile_kind and self._profile_kind == ("decode" if all(len(s.tokens) == 1 for s in batch) else "prefill"):
            self._profile_seen += 1
            if self._profile_due(self._profile_seen):
                self._profiled_step(entries)
                n = sum(1 for s in batch if s.sample)
                return self.sampler.download(n) if n else None
        self.engine.step(entries, logits=False)
        n = sum(1 for s in batch if s.sample)
        return self.sampler.download(n) if n else None

    def _profile_due(self, count: int) -> bool:
        return self._profile_every == 1 or count % self._profile_every == 1

    def _profiled_step(self, entries) -> None:
        from .. import ops
        graphs, self.engine.cuda_graphs = self.engine.cuda_graphs, False
        prof = ops.SegmentProfiler()
        old = ops.set_profiler(prof)
        prof.begin()
        try:
            self.engine.step(entries, logits=False)
        finally:
            ops.set_profiler(old)
            self.engine.cuda_graphs = graphs
        self._profile_runs.append(prof.summary())

    def profile_report(self) -> List[str]:
        """Lines of the mean over the profiled steps, by kernel family (empty without REINFER_B200_STEP_PROFILE)."""
        if not self._profile_runs:
            return []
        from .. import measure
        mean: Dict = {}
        for run in self._profile_runs:
            for name, d in run.items():
                m = mean.setdefault(name, {"n": 0, "us": 0.0, "tflops": 0.0, "gbs": 0.0})
                for k in m:
                    m[k] += d[k] / len(self._profile_runs)
        for m in mean.values():
            m["n"] = int(round(m["n"]))
        hbm, tf, _, src = measure.peaks()
        return [f"-- mean of {len(self._profile_runs)} eager {self._profile_kind} steps by kernel family (peaks {src}) --"] + \
            measure.segment_table(mean, hbm, tf)

    def _launch_ahead(self, batch):
        """If the step after `batch` (which is launched, not read) is sure to be "the same requests, one token
        each", launch it now.  Returns (its requests, its tokens on their way) or None."""
        if not self.engine.cuda_graphs or self.scheduler.waiting or len(batch) != len(self.scheduler.running):
            return None
        limit = self.max_model_len
        for s in batch:
            r = s.request
            if not s.sample or r.state != RUNNING or len(r.output) + 1 >= r.params.max_tokens or \
                    (limit and r.total_len + 2 >= limit):
                return None
        if self._profile_kind == "decode":
            if self._profile_due(self._profile_seen + 1):
                return None                             # the next decode step is one to profile: it takes the ordinary way
            self._profile_seen += 1
        handle = self.engine.prepare_ahead([s.request.request_id for s in batch])
        if handle is None:
            return None
        self.engine.step_ahead(handle, None, logits=False)
        self.steps_launched_ahead += 1
        return [s.request for s in batch], self.sampler.download(len(batch))

    def generate(self, prompt_token_ids: Union[Sequence[int], Sequence[Sequence[int]]],
                 sampling_params: Union[None, SamplingParams, Sequence[SamplingParams]] = None) -> List[RequestOutput]:
        """Generate for one prompt or a list of prompts (token ids); results in the order given."""
        prompts = prompt_token_ids
        if prompts and isinstance(prompts[0], int):
            prompts = [prompts]
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            plist = [sampling_params or SamplingParams()] * len(prompts)
        else:
            plist = list(sampling_params)
            if len(plist) != len(prompts):
                raise ValueError("one SamplingParams per prompt")
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, plist)]
        t0 = time.perf_counter()
        steps = 0
        while self.has_work():
            self.step()
            steps += 1
        dt = time.perf_counter() - t0
        outs = []
        for rid in ids:
            r = self.requests.pop(rid)
            outs.append(RequestOutput(rid, r.prompt, list(r.output), r.finish_reason, r.preemptions))
        n_out = sum(len(o.token_ids) for o in outs)
        self.last_stats = {"seconds": dt, "steps": steps, "generated": n_out,
                           "tok_s": n_out / dt if dt > 0 else 0.0,
                           "preemptions": self.scheduler.stats["preemptions"]}
        return outs
