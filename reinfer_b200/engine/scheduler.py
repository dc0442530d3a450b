"""Continuous batching above the step function: admits requests, cuts prompts into
portions under a token budget, decodes, finishes and frees.  Pure host logic: it asks the
cache manager for page counts and never touches a device, so it is tested with a fake
step function.

Decisions, after the reference's scheduler (crates/scheduler/src/batch.rs:69-101
`select_batch`; policy.rs:30-63; req.rs:121-405; bin/reinfer/src/sched_loop.rs:756-1079):
  * every decoding request gets its one token first, in arrival order; what is left of
    `max_batch_tokens` goes to prompts: first to requests already in the middle of their
    prompt, then to waiting requests in queue order (resumed requests stand at the front),
    each portion = min(rest of the prompt, max_chunk, rest of the budget), cut anywhere;
  * a waiting request is admitted when a slot is free and the free pages cover its whole
    prompt and one more token, the pages still promised to prompts in progress, and one
    page per running request (head room for their next tokens); so an admitted prompt can
    always be finished;
  * when pages run out for the decoding requests, the newest arrival is preempted first
    (requests that were preempted before come last): its pages and slot are given back and
    it returns to the FRONT of the waiting queue.  On resume it recomputes prompt + tokens
    generated so far and then goes on generating (the reference restarts the request and
    regenerates, req.rs:346-357);
  * a request that cannot fit into an empty pool finishes with reason "too_long";
  * after sampling: stop token or stop sequence -> EOS -> max_tokens, in that order; a stop or EOS
    token is consumed, not emitted; exactly max_tokens tokens are emitted otherwise
    (req.rs:294-315).  A stop sequence is a sequence of token ids that ends the output stream
    (stop.rs:1-13: matched on the raw token stream, the moment its last token is drawn); the
    tokens of it that were emitted before are taken back from the output as well;
  * abort is idempotent and releases exactly once (req.rs:330-339);
  * optionally (`admission=`) a waiting request must also pass the reference's estimate of the
    working set's peak (engine/admission.py); a request is never held back by it while nothing
    else runs, so the queue always moves.
Scheduling is a pure function of (arrival order, parameters, pool size).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams
from .admission import EstimateAdmission

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
    request_id: Hashable
    prompt: List[int]
    params: SamplingParams
    arrival: int = 0
    seed: int = 0
    state: str = WAITING
    output: List[int] = field(default_factory=list)
    num_computed: int = 0                   # tokens of (prompt + output) whose keys are cached
    preemptions: int = 0
    finish_reason: Optional[str] = None

    @property
    def all_tokens(self) -> List[int]:
        return self.prompt + self.output

    def tokens_from(self, start: int, n: int) -> List[int]:
        """Tokens start..start+n-1 of prompt + output, without building the joined list."""
        lp = len(self.prompt)
        if start >= lp:
            return self.output[start - lp:start - lp + n]
        if start + n <= lp:
            return self.prompt[start:start + n]
        return self.prompt[start:] + self.output[:start + n - lp]

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def in_prefill(self) -> bool:
        """True while tokens other than the newest one are still to be computed."""
        return self.total_len - self.num_computed > 1 or not self.output


def _stop_sequence_match(sequences, output: List[int], token: int) -> Optional[int]:
    """If output + [token] ends with one of the sequences: how many tokens of it are already in the output (the
    longest such sequence wins, so that all of it is taken back).  Empty sequences never match."""
    best = None
    for seq in sequences:
        n = len(seq)
        if n and seq[-1] == token and n - 1 <= len(output) and list(seq[:-1]) == output[len(output) - (n - 1):]:
            best = n - 1 if best is None else max(best, n - 1)
    return best


@dataclass
class Scheduled:
    request: Request
    start: int                              # first position computed in this step
    tokens: List[int]
    sample: bool                            # the logits of the last token are wanted


@dataclass
class SchedulerOutput:
    batch: List[Scheduled]
    preempted: List[Request]
    finished: List[Request]                 # finished without running (too long, aborted)


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch_tokens: int = 2048, max_chunk: Optional[int] = None,
                 eos_token_ids: Sequence[int] = (), max_model_len: Optional[int] = None,
                 release: Optional[Callable[[Hashable], None]] = None,
                 admission: Optional[EstimateAdmission] = None):
        if max_batch_tokens <= 0:
            raise ValueError("max_batch_tokens must be positive")
        self.cache = cache
        self.max_batch_tokens = int(max_batch_tokens)
        self.max_chunk = int(max_chunk) if max_chunk else self.max_batch_tokens
        self.eos = tuple(eos_token_ids)
        self.max_model_len = max_model_len
        self._release = release or (lambda rid: cache.release(rid) if rid in cache else None)
        self.admission = admission
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self._arrivals = 0
        self.stats = {"preemptions": 0, "steps": 0, "scheduled_tokens": 0}

    # ---- arrivals and departures ----------------------------------------------------------
    def add(self, request: Request) -> None:
        request.params.validate()
        if not request.prompt:
            raise ValueError(f"request {request.request_id!r} has an empty prompt")
        request.arrival = self._arrivals
        self._arrivals += 1
        request.state = WAITING
        self.waiting.append(request)

    def abort(self, request_id) -> Optional[Request]:
        for r in list(self.running):
            if r.request_id == request_id:
                self.running.remove(r)
                self._finish(r, "abort")
                return r
        for r in list(self.waiting):
            if r.request_id == request_id:
                self.waiting.remove(r)
                self._finish(r, "abort")
                return r
        return None

    def fail(self, request: Request, reason: str = "error") -> None:
        """The step that ran this request failed: it ends with `reason` and gives back what it holds."""
        if request in self.running:
            self.running.remove(request)
        elif request in self.waiting:
            self.waiting.remove(request)
        self._finish(request, reason)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _finish(self, r: Request, reason: str) -> None:
        if r.state == FINISHED:
            return
        r.state = FINISHED
        r.finish_reason = reason
        self._release(r.request_id)
        if self.admission is not None and reason in ("stop", "eos", "length"):
            self.admission.finished(len(r.output))

    # ---- one scheduling decision ------------------------------------------------------------
    def schedule(self) -> SchedulerOutput:
        cm = self.cache
        ps = cm.page_size
        preempted: List[Request] = []
        finished: List[Request] = []

        def pages_more(r: Request, upto: int) -> int:
            return cm.pages_needed(r.request_id, upto) if r.request_id in cm else cm.pages_for(upto)

        while True:
            budget = self.max_batch_tokens
            batch: List[Scheduled] = []
            decoding = sorted((r for r in self.running if not r.in_prefill), key=lambda r: r.arrival)
            prefilling = sorted((r for r in self.running if r.in_prefill), key=lambda r: r.arrival)
            # 1. every decoding request needs room for one more token; preempt the newest
            #    arrival (requests preempted before come last) while that does not fit
            need = sum(pages_more(r, r.num_computed + 1) for r in decoding)
            if need > cm.free_pages():
                victims = sorted(self.running, key=lambda r: (r.preemptions > 0, -r.arrival))
                v = victims[0]
                if len(self.running) == 1:
                    # alone in the pool and still too large: it can never go on
                    self.running.remove(v)
                    self._finish(v, "too_long")
                    finished.append(v)
                else:
                    self._preempt(v)
                    preempted.append(v)
                continue
            free = cm.free_pages()
            # who decodes is decided by arrival; in the batch they stand longest first (the attention kernel starts
            # its CTAs in the order of the entries, and the ones with most keys should begin first)
            for r in sorted(decoding[:budget], key=lambda r: (-r.num_computed, r.arrival)):
                free -= pages_more(r, r.num_computed + 1)
                batch.append(Scheduled(r, r.num_computed, r.tokens_from(r.num_computed, 1), True))
                budget -= 1

            # 2. prompts in progress: their pages were promised at admission
            promised = 0
            for r in prefilling:
                rest = r.total_len - r.num_computed
                room = (len(cm.table(r.request_id, 0)) * ps if r.request_id in cm and cm.groups else 0) \
                    + free * ps - r.num_computed
                n = min(rest, self.max_chunk, budget, room)
                if n > 0:
                    free -= pages_more(r, r.num_computed + n)
                    batch.append(Scheduled(r, r.num_computed, r.tokens_from(r.num_computed, n), n == rest))
                    budget -= n
                promised += max(0, pages_more(r, r.total_len + 1) - (pages_more(r, r.num_computed + n) if n > 0 else 0))

            # 3. the waiting queue, in order; nothing is admitted in a step that preempted
            admitted = 0
            first_portions = 0
            taken: List[Request] = []
            while self.waiting and budget > 0 and not preempted:
                r = self.waiting[0]
                limit = self.max_model_len
                if r.params.max_tokens == 0:
                    self.waiting.popleft()
                    self._finish(r, "length")
                    finished.append(r)
                    continue
                if cm.pages_for(r.total_len + 1) > cm.total_pages() or (limit and r.total_len + 1 > limit):
                    self.waiting.popleft()
                    self._finish(r, "too_long")
                    finished.append(r)
                    continue
                if cm.free_slots() - admitted <= 0:
                    break
                reserve = len(self.running) + admitted          # head room: one page per running request
                if cm.pages_for(r.total_len + 1) + reserve + promised > free:
                    break
                rest = r.total_len - r.num_computed
                n = min(rest, self.max_chunk, budget)
                if self.admission is not None and (self.running or taken):
                    live = [(len(q.prompt), len(q.output), q.num_computed, q.params.max_tokens) for q in self.running + taken]
                    used = (cm.total_pages() - cm.free_pages()) * ps
                    if not self.admission.admits(live, (len(r.prompt), len(r.output), r.num_computed, r.params.max_tokens),
                                                 used_tokens=used, portion=self.max_chunk, first_portion=n,
                                                 first_portions_so_far=first_portions):
                        break
                first_portions += n
                taken.append(r)
                self.waiting.popleft()
                free -= cm.pages_for(n)
                promised += cm.pages_for(r.total_len + 1) - cm.pages_for(n)
                batch.append(Scheduled(r, r.num_computed, r.tokens_from(r.num_computed, n), n == rest))
                budget -= n
                admitted += 1
            if not batch and self.running and not preempted:
                # nobody can move (pages are held by half-computed prompts): free the newest
                v = sorted(self.running, key=lambda r: (r.preemptions > 0, -r.arrival))[0]
                if len(self.running) == 1:
                    self.running.remove(v)
                    self._finish(v, "too_long")
                    finished.append(v)
                else:
                    self._preempt(v)
                    preempted.append(v)
                continue
            break
        for s in batch:
            if s.request.state == WAITING:
                s.request.state = RUNNING
                self.running.append(s.request)
        self.stats["steps"] += 1
        self.stats["scheduled_tokens"] += sum(len(s.tokens) for s in batch)
        return SchedulerOutput(batch, preempted, finished)

    def schedule_decode(self, requests: Sequence[Request]) -> List[Scheduled]:
        """The batch of a step that is already running: these running requests, each with the one token drawn
        for it last.  (The entry point launches such a step before it has read the step before, when that one
        was sure to be followed by "everybody decodes again"; requests that turned out to end there are simply
        not named here, and their rows of the running step are dropped.)"""
        batch = []
        for r in requests:
            if r.state != RUNNING or r.in_prefill:
                raise ValueError(f"request {r.request_id!r} is not decoding")
            batch.append(Scheduled(r, r.num_computed, r.tokens_from(r.num_computed, 1), True))
        self.stats["steps"] += 1
        self.stats["scheduled_tokens"] += len(batch)
        return batch

    def _preempt(self, r: Request) -> None:
        self.running.remove(r)
        self._release(r.request_id)
        r.num_computed = 0
        r.preemptions += 1
        r.state = WAITING
        self.waiting.appendleft(r)
        self.stats["preemptions"] += 1

    # ---- after the step ---------------------------------------------------------------------
    def update(self, batch: Sequence[Scheduled], sampled: Dict[Hashable, int]) -> List[Request]:
        """Record what the step computed and the tokens drawn for the entries that wanted one.
        Returns the requests that finished."""
        done: List[Request] = []
        for s in batch:
            r = s.request
            if r.state != RUNNING:
                continue                                    # aborted meanwhile
            r.num_computed = s.start + len(s.tokens)
            if not s.sample:
                continue
            tok = sampled[r.request_id]
            p = r.params
            if tok < 0:
                reason = "no_token"                         # no finite logit
            elif tok in p.stop_token_ids:
                reason = "stop"
            elif (cut := _stop_sequence_match(p.stop_sequences, r.output, tok)) is not None:
                reason = "stop"
                del r.output[len(r.output) - cut:]
            elif tok in self.eos and not p.ignore_eos:
                reason = "eos"
            else:
                r.output.append(tok)
                reason = "length" if len(r.output) >= p.max_tokens else None
            if reason is None and self.max_model_len and r.total_len >= self.max_model_len:
                reason = "length"
            if reason is not None:
                self.running.remove(r)
                self._finish(r, reason)
                done.append(r)
        return done
