"""An optional admission policy for the scheduler: admit a waiting request only if the
estimated peak of the whole working set fits the cache pool, so that requests which will
grow while they decode are not admitted into a pool they would later be preempted from.

The estimate is the reference's (crates/scheduler/src/admission.rs:72-87 per request,
:120-148 output-length average and peak, :211-253 the gates):

  * a request's footprint now: `a = prompt + generated + 1`;
  * what it is still expected to add: `b = max_new` when the pool is busy (occupancy at or
    above `busy_ratio`), else `min(max_new, max(ceil(1.1 * generated), average))`, where
    `average` is a running average of the output lengths of finished requests; plus 16 tokens
    of slack; plus, while its prompt is still being computed in portions,
    `ceil(rest of the prompt / portion) * (max_waiting + 1)`;
  * the peak of a set: sort by `b` descending; `max over k of b_k * k + sum of a_j for j <= k`
    (the k requests that live longest all hold `b_k` more tokens when the k-th ends);
  * gates, in order: number of requests; the totals (busy: sum a + sum b, else each sum alone);
    the peak; and the sum of the first portions admitted in one step.

Pure host arithmetic on integers; the scheduler keeps its own page-exact rule beside it (that
rule guarantees that an admitted prompt can be finished, this one keeps preemptions rare).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

OUTPUT_SLACK = 16                  # tokens added to every request's expected growth
AVERAGE_START = 2048.0             # the output-length average before any request has finished
AVERAGE_FLOOR = 64.0


class OutputLengthAverage:
    """Running average of finished requests' output lengths.  An output longer than the average
    moves it slowly (0.9 of the old value is kept), a shorter one faster (0.6), and it never falls
    below the floor (crates/scheduler/src/admission.rs:89-133)."""

    def __init__(self, start: float = AVERAGE_START, floor: float = AVERAGE_FLOOR):
        self.value = float(start)
        self.floor = float(floor)
        self.keep = 0.6

    def observe(self, output_len: int) -> float:
        self.keep = 0.9 if output_len > self.value else 0.6
        self.value = max(self.floor, self.keep * self.value + (1.0 - self.keep) * float(output_len))
        return self.value


@dataclass(frozen=True)
class Footprint:
    now: int                       # a: tokens the request holds once its prompt and outputs so far are cached
    growth: int                    # b: tokens it is expected to add before it ends


def footprint(prompt_len: int, generated: int, max_new: int, *, busy: bool, average: float,
              rest_of_prompt: int = 0, portion: int = 0, max_waiting: int = 0, shared: int = 0) -> Footprint:
    now = max(prompt_len + generated + 1, shared + 1)
    if busy:
        growth = max_new
    else:
        growth = min(max_new, max(math.ceil(1.1 * generated), int(round(average))))
    growth += OUTPUT_SLACK
    if rest_of_prompt > 0 and portion > 0:
        growth += -(-rest_of_prompt // portion) * (max_waiting + 1)
    return Footprint(now, growth)


def peak_tokens(working: Sequence[Footprint]) -> int:
    """The most tokens the set is expected to hold at any time."""
    peak = held = 0
    for k, f in enumerate(sorted(working, key=lambda f: -f.growth), start=1):   # stable: ties keep their order
        held += f.now
        peak = max(peak, f.growth * k + held)
    return peak


@dataclass
class AdmissionLimits:
    pool_tokens: int               # pages of the pool x page size
    max_requests: int
    max_batch_tokens: int
    portions_factor: int = 2       # the first portions of one step may sum to this many batches
    busy_ratio: float = 0.8
    max_waiting: int = 16


PEAK, COUNT, FIRST_PORTIONS = "peak", "count", "first_portions"


def refusal(working: Sequence[Footprint], limits: AdmissionLimits, *, busy: bool,
            first_portion: Optional[int] = None, first_portions_so_far: int = 0) -> Optional[str]:
    """None if the set (the request under review included) is admitted, else which gate refused it."""
    if len(working) > limits.max_requests:
        return COUNT
    now, growth = sum(f.now for f in working), sum(f.growth for f in working)
    fits = now + growth <= limits.pool_tokens if busy else max(now, growth) <= limits.pool_tokens
    if not fits or peak_tokens(working) > limits.pool_tokens:
        return PEAK
    if first_portion is not None and \
            first_portions_so_far + first_portion > limits.max_batch_tokens * limits.portions_factor:
        return FIRST_PORTIONS
    return None


class EstimateAdmission:
    """What the scheduler asks: `admits(running, candidate, ...)` before it takes a request from the
    waiting queue, `finished(output_len)` when a request ends by itself."""

    def __init__(self, limits: AdmissionLimits):
        self.limits = limits
        self.average = OutputLengthAverage()
        self.refusals = {PEAK: 0, COUNT: 0, FIRST_PORTIONS: 0}

    def busy(self, used_tokens: int) -> bool:
        lim = self.limits
        return lim.pool_tokens > 0 and lim.busy_ratio <= 1.0 and used_tokens / lim.pool_tokens >= lim.busy_ratio

    def footprint_of(self, prompt_len: int, generated: int, computed: int, max_new: int, busy: bool,
                     portion: int) -> Footprint:
        rest = max(0, prompt_len - computed)
        return footprint(prompt_len, generated, max_new, busy=busy,
                         average=self.average.value, rest_of_prompt=rest if rest > portion else 0,
                         portion=portion, max_waiting=self.limits.max_waiting)

    def admits(self, running: List[Tuple[int, int, int, int]], candidate: Tuple[int, int, int, int], *,
               used_tokens: int, portion: int, first_portion: int, first_portions_so_far: int) -> bool:
        """running / candidate: (prompt length, tokens generated, tokens cached, max new tokens)."""
        busy = self.busy(used_tokens)
        working = [self.footprint_of(p, g, c, m, busy, portion) for p, g, c, m in running + [candidate]]
        why = refusal(working, self.limits, busy=busy, first_portion=first_portion,
                      first_portions_so_far=first_portions_so_far)
        if why is not None:
            self.refusals[why] += 1
        return why is None

    def finished(self, output_len: int) -> None:
        self.average.observe(output_len)
