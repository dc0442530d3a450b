"""The optional admission estimate (reinfer_b200/engine/admission.py): its arithmetic against the
reference's formulas and worked examples (crates/scheduler/src/admission.rs:72-148, 211-253 and the
cases of its own tests, :283-440, read as text), and what the scheduler does with it.  No GPU."""
import random

from reinfer_b200.engine.admission import (AdmissionLimits, COUNT, EstimateAdmission, FIRST_PORTIONS, Footprint,
                                           OutputLengthAverage, PEAK, footprint, peak_tokens, refusal)
from test_scheduler import Loop, req


def test_footprint_now_and_growth():
    assert footprint(100, 0, 64, busy=False, average=2048).now == 101
    assert footprint(100, 7, 64, busy=False, average=2048).now == 108
    assert footprint(100, 7, 64, busy=False, average=2048, shared=200).now == 201
    # idle: min(max_new, max(1.1 x generated, average)) + 16
    assert footprint(8, 0, 64, busy=False, average=2048).growth == 80
    assert footprint(8, 20, 300, busy=False, average=2048).growth == 316
    assert footprint(8, 20, 300, busy=False, average=10).growth == 22 + 16
    # busy: the pessimistic max_new + 16
    assert footprint(8, 20, 300, busy=True, average=10).growth == 316
    # a prompt still computed in portions lives longer: ceil(rest / portion) x (max_waiting + 1)
    f = footprint(1000, 0, 64, busy=False, average=2048, rest_of_prompt=700, portion=256, max_waiting=16)
    assert f.growth == 64 + 16 + 3 * 17


def test_output_length_average():
    avg = OutputLengthAverage()
    assert avg.value == 2048
    v = avg.observe(100)                              # shorter: 0.6 of the old value is kept
    assert abs(v - (0.6 * 2048 + 0.4 * 100)) < 1e-9 and avg.keep == 0.6
    v2 = avg.observe(5000)                            # longer: 0.9 is kept
    assert abs(v2 - (0.9 * v + 0.1 * 5000)) < 1e-9 and avg.keep == 0.9
    for _ in range(100):
        avg.observe(1)
    assert avg.value == 64                            # the floor


def brute_peak(working):
    """The definition: the requests end in the order of their growth; when the k-th longest-living one is
    about to end, it and the k-1 that outlive it each hold growth_k more than now."""
    order = sorted(working, key=lambda f: -f.growth)
    best = 0
    for k in range(1, len(order) + 1):
        best = max(best, sum(f.now for f in order[:k]) + order[k - 1].growth * k)
    return best


def test_peak_tokens():
    assert peak_tokens([]) == 0
    assert peak_tokens([Footprint(10, 5)]) == 15
    assert peak_tokens([Footprint(10, 5), Footprint(3, 9)]) == 23
    rng = random.Random(0)
    for _ in range(200):
        w = [Footprint(rng.randint(1, 500), rng.randint(0, 300)) for _ in range(rng.randint(1, 9))]
        assert peak_tokens(w) == brute_peak(w)
        assert peak_tokens(w) <= sum(f.now + f.growth for f in w)         # never above the totals
        assert peak_tokens(w) >= max(f.now + f.growth for f in w)


def test_gates_in_order():
    lim = AdmissionLimits(pool_tokens=1000, max_requests=2, max_batch_tokens=100)
    three = [Footprint(10, 10)] * 3
    assert refusal(three, lim, busy=False) == COUNT
    assert refusal([Footprint(600, 100), Footprint(300, 100)], lim, busy=False) == PEAK    # 100 x 2 + 900 > 1000
    assert refusal([Footprint(500, 100), Footprint(300, 100)], lim, busy=False) is None
    # busy: the totals are summed
    assert refusal([Footprint(500, 150), Footprint(300, 100)], lim, busy=True) == PEAK
    assert refusal([Footprint(400, 100), Footprint(300, 100)], lim, busy=True) is None
    ok = [Footprint(100, 10)]
    assert refusal(ok, lim, busy=False, first_portion=150, first_portions_so_far=100) == FIRST_PORTIONS
    assert refusal(ok, lim, busy=False, first_portion=100, first_portions_so_far=100) is None


def test_scheduler_holds_back_what_would_not_fit_at_its_peak():
    """A pool of 160 tokens and three requests that end at 60 tokens each.  By pages alone all three are admitted
    at once (their prompts fit) and one is preempted when they grow; with the estimate (2 x 64 + 26 fits, 3 x 64 + 39
    does not) the third waits until one has ended, and nothing is preempted."""
    def run(admission):
        loop = Loop(40, page_size=4, max_seqs=4, max_batch_tokens=64, admission=admission)
        reqs = [req(f"r{i}", 12, max_tokens=48, ignore_eos=True) for i in range(3)]
        for r in reqs:
            loop.s.add(r)
        loop.run()
        first_steps = {}
        for n, out in enumerate(loop.history):
            for s in out.batch:
                first_steps.setdefault(s.request.request_id, n)
        return loop, first_steps, reqs

    plain, when_plain, reqs_plain = run(None)
    assert set(when_plain.values()) == {0} and plain.s.stats["preemptions"] >= 1
    est = EstimateAdmission(AdmissionLimits(pool_tokens=160, max_requests=4, max_batch_tokens=64))
    est.average.value = 48.0
    held, when, reqs_held = run(est)
    assert when["r0"] == 0 and when["r1"] == 0 and when["r2"] > 40
    assert held.s.stats["preemptions"] == 0
    assert est.refusals[PEAK] >= 1
    # every request ran to its end either way, with the same tokens
    for a, b in zip(reqs_plain, reqs_held):
        assert len(a.output) == 48 and a.output == b.output
    # the estimate has heard of the three that ended
    assert est.average.value == 64.0                  # 48 each time, held up by the floor


def test_a_request_alone_is_never_held_back():
    """The estimate would refuse it (the average says 2,048 more tokens), but nothing else runs: it goes."""
    est = EstimateAdmission(AdmissionLimits(pool_tokens=32, max_requests=4, max_batch_tokens=64))
    loop = Loop(8, page_size=4, max_seqs=4, max_batch_tokens=64, admission=est)
    loop.s.add(req("a", 10, max_tokens=8, ignore_eos=True))
    loop.s.add(req("b", 10, max_tokens=8, ignore_eos=True))
    loop.run()
    assert loop.history[0].batch and loop.history[0].batch[0].request.request_id == "a"
    assert est.refusals[PEAK] >= 1                    # b waited for a
    assert loop.s.stats["preemptions"] == 0
