"""The Python entry point: `LLM(model_dir).generate(prompt_token_ids, SamplingParams)`.
It joins the scheduler, the engine's step function and the GPU sampler in the loop that
the reference runs in bin/reinfer/src/sched_loop.rs:564-587, 691-695 (admit and schedule,
step, sample, finish), with prompts' portions and decoded tokens in ONE step call instead
of separate engine calls.  Token ids in, token ids out: the tokenizer is not part of this
engine.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..config.registry import resolve_eos
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, request_seed
from .admission import AdmissionLimits, EstimateAdmission
from .engine import Engine, EngineError, StepEntry
from .scheduler import Request, Scheduler


@dataclass
class RequestOutput:
    request_id: Hashable
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: Optional[str]
    preemptions: int = 0


def penalty_window(request: Request, last_n: int) -> List[int]:
    """The tokens that the repeat, frequency and presence penalties look at: the last `last_n` tokens the
    request has SAMPLED, never its prompt (crates/cuda/src/sampler.rs:109-111 and :369: the history is
    fed by `history.push(token)` after each draw).  A preempted request keeps its output, so the window
    is the same after it resumes."""
    return request.output[-last_n:] if last_n > 0 else []


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
        self.sampler = Sampler(engine.vocab_size, engine.cache.max_seqs, engine.device)
        self._next_id = 0
        self.requests: Dict[Hashable, Request] = {}
        self.last_stats: Dict[str, float] = {}
        self._ahead = None                      # tables of the next step, built while the device was busy
        self.ahead_used = 0                     # steps that ran on tables prepared one step ahead
        self.ahead_discarded = 0                # prepared tables that the next decision did not match

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
        return self.scheduler.has_work()

    def step(self) -> List[Request]:
        """One scheduler decision, one engine step, one sampler launch.  Returns the requests
        that finished in it.

        While the device runs the step, the host already builds the next step's tables under the guess
        that the same requests simply go on decoding (`Engine.prepare_ahead`); if the next decision is
        exactly that, only the sampled token ids are filled in before the replay."""
        out = self.scheduler.schedule()
        finished = list(out.finished)
        if not out.batch:
            return finished
        ahead, self._ahead = self._ahead, None
        rids = tuple(s.request.request_id for s in out.batch)
        sampling = [s.request for s in out.batch if s.sample]
        sampled: Dict[Hashable, int] = {}
        try:
            if ahead is not None and ahead[1] == rids and all(len(s.tokens) == 1 and s.sample for s in out.batch):
                self.ahead_used += 1
                logits = self.engine.step_ahead(ahead, [s.tokens[0] for s in out.batch])
            else:
                if ahead is not None:
                    self.ahead_discarded += 1           # (its pages stay with their requests)
                entries = [StepEntry(s.request.request_id, s.tokens, [len(s.tokens) - 1] if s.sample else [])
                           for s in out.batch]
                logits = self.engine.step(entries)
            if sampling:
                n = self.sampler.launch(logits, [r.params for r in sampling], [r.seed for r in sampling],
                                        [len(r.output) for r in sampling],
                                        [(lambda k, r=r: penalty_window(r, k)) for r in sampling])
                # the device is busy: prepare the next step if it is likely to be these requests again
                if len(sampling) == len(out.batch) and not self.scheduler.waiting and \
                        all(len(r.output) + 1 < r.params.max_tokens for r in sampling):
                    self._ahead = self.engine.prepare_ahead(rids)
                toks = self.sampler.fetch(n)
                sampled = {r.request_id: t for r, t in zip(sampling, toks)}
                self.engine.check_status()              # the tokens have arrived: the step's kernels are over
        except EngineError:
            # a kernel gave up (or the engine refused the step): the requests of this step end with "error" and
            # give back their pages; the engine refuses further steps until `engine.clear_status()`
            self._ahead = None
            for s in out.batch:
                self.scheduler.fail(s.request)
            raise
        finished += self.scheduler.update(out.batch, sampled)
        return finished

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
