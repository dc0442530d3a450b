"""The scheduler's decisions with a fake step function whose token is a pure function of
(request, position) - no GPU.  (The idea of the reference's MockExecutor,
bin/reinfer/src/sched_loop.rs:1594-1781.)"""
import zlib

import pytest

from reinfer_b200.cache import CacheManager
from reinfer_b200.engine.scheduler import FINISHED, Request, Scheduler
from reinfer_b200.parts.base import PagedKVSpec
from reinfer_b200.sampling import SamplingParams

SPEC = {"l0": PagedKVSpec(2, 16)}


def fake_token(rid, position, vocab=1000):
    """The same in every process (the built-in hash of a string is not)."""
    return (zlib.crc32(f"{rid}:{position}".encode()) % (vocab - 10)) + 10


class Loop:
    """What LLM.step does, with the engine replaced by page bookkeeping and a fake sampler."""

    def __init__(self, num_pages, page_size=4, max_seqs=4, **kw):
        self.cm = CacheManager(SPEC, {}, page_size, num_pages, max_seqs)
        self.s = Scheduler(self.cm, **kw)
        self.history = []

    def step(self):
        out = self.s.schedule()
        for s in out.batch:
            rid = s.request.request_id
            if rid not in self.cm:
                self.cm.admit(rid)
            assert s.start == self.cm.length(rid)
            self.cm.reserve(rid, s.start + len(s.tokens))
        for s in out.batch:
            self.cm.commit(s.request.request_id, s.start + len(s.tokens))
        sampled = {s.request.request_id: fake_token(s.request.request_id, s.start + len(s.tokens))
                   for s in out.batch if s.sample}
        done = self.s.update(out.batch, sampled)
        self.cm.check()
        self.history.append(out)
        return out, done

    def run(self, limit=10000):
        n = 0
        while self.s.has_work():
            self.step()
            n += 1
            assert n < limit, "the scheduler does not come to an end"
        return n


def req(rid, n_prompt, **kw):
    return Request(rid, list(range(1, n_prompt + 1)), SamplingParams(**kw))


def test_budget_decode_first_and_portions_cut_anywhere():
    lp = Loop(num_pages=200, max_seqs=4, max_batch_tokens=16)
    lp.s.add(req("a", 40, max_tokens=3))
    out, _ = lp.step()
    assert [(s.request.request_id, s.start, len(s.tokens), s.sample) for s in out.batch] == [("a", 0, 16, False)]
    lp.s.add(req("b", 5, max_tokens=3))
    out, _ = lp.step()                       # a goes on first (in progress), nothing is left for b
    assert [(s.request.request_id, s.start, len(s.tokens)) for s in out.batch] == [("a", 16, 16)]
    out, _ = lp.step()                       # a's last 8 tokens (sampled), b's whole prompt beside it
    assert [(s.request.request_id, s.start, len(s.tokens), s.sample) for s in out.batch] == \
        [("a", 32, 8, True), ("b", 0, 5, True)]
    lp.s.add(req("c", 30, max_tokens=2))
    out, _ = lp.step()                       # both decode (one token each) first, 14 tokens of c after them
    assert [(s.request.request_id, len(s.tokens)) for s in out.batch] == [("a", 1), ("b", 1), ("c", 14)]
    assert sum(len(s.tokens) for s in out.batch) == 16
    lp.run()
    assert lp.cm.free_pages() == 200 and lp.cm.free_slots() == 4


def test_exact_output_lengths_and_stop_order():
    lp = Loop(num_pages=100, max_batch_tokens=64)
    a, b, c = req("a", 7, max_tokens=5), req("b", 3, max_tokens=50), req("c", 3, max_tokens=50)
    third_b = fake_token("b", 3 + 2)
    b.params.stop_token_ids = (third_b,)
    lp.s.eos = (fake_token("c", 3 + 1),)
    for r in (a, b, c):
        lp.s.add(r)
    lp.run()
    assert len(a.output) == 5 and a.finish_reason == "length"
    assert a.output == [fake_token("a", 7 + i) for i in range(5)]
    assert len(b.output) == 2 and b.finish_reason == "stop"          # the stop token is consumed, not emitted
    assert len(c.output) == 1 and c.finish_reason == "eos"
    d = req("d", 3, max_tokens=4, ignore_eos=True)
    lp.s.eos = (fake_token("d", 3),)
    lp.s.add(d)
    lp.run()
    assert len(d.output) == 4 and d.finish_reason == "length"


def test_slots_bound_the_running_set():
    lp = Loop(num_pages=100, max_seqs=2, max_batch_tokens=64)
    for i in range(5):
        lp.s.add(req(i, 4, max_tokens=3))
    out, _ = lp.step()
    assert len(out.batch) == 2 and len(lp.s.running) == 2 and len(lp.s.waiting) == 3
    lp.run()
    assert all(h.batch for h in lp.history)


def test_preemption_newest_first_resumes_and_outputs_do_not_change():
    def outputs(num_pages):
        lp = Loop(num_pages=num_pages, page_size=4, max_seqs=4, max_batch_tokens=32)
        rs = [req(i, 6 + i, max_tokens=20) for i in range(3)]
        for r in rs:
            lp.s.add(r)
        lp.run()
        assert lp.cm.free_pages() == num_pages
        return rs, lp

    calm, _ = outputs(100)
    tight, lp = outputs(14)                   # 3 requests x up to 28 tokens = 21 pages wanted, 14 exist
    assert lp.s.stats["preemptions"] > 0
    assert [r.output for r in tight] == [r.output for r in calm]
    assert all(r.finish_reason == "length" for r in tight)
    first = next(h for h in lp.history if h.preempted)
    assert first.preempted[0].request_id == 2                        # the newest arrival goes first
    assert tight[0].preemptions == 0
    # the victim came back at the front of the queue and recomputed prompt + what it had generated
    k = lp.history.index(first)
    later = next(s for h in lp.history[k + 1:] for s in h.batch if s.request.request_id == 2)
    assert later.start == 0 and len(later.tokens) > len(tight[2].prompt) - 1


def test_request_that_can_never_fit_finishes_too_long():
    lp = Loop(num_pages=4, page_size=4, max_batch_tokens=64)
    big, ok = req("big", 40, max_tokens=2), req("ok", 5, max_tokens=2)
    lp.s.add(big); lp.s.add(ok)
    lp.run()
    assert big.finish_reason == "too_long" and big.output == []
    assert ok.finish_reason == "length" and len(ok.output) == 2
    grow = req("grow", 10, max_tokens=50)                            # fits at first, outgrows the pool alone
    lp.s.add(grow)
    lp.run()
    assert grow.finish_reason == "too_long" and 0 < len(grow.output) < 50
    assert lp.cm.free_pages() == 4


def test_abort_is_idempotent_and_frees_once():
    lp = Loop(num_pages=50, max_batch_tokens=8)
    a, b = req("a", 20, max_tokens=10), req("b", 4, max_tokens=10)
    lp.s.add(a); lp.s.add(b)
    lp.step()
    assert lp.s.abort("a") is a and a.state == FINISHED and a.finish_reason == "abort"
    assert lp.s.abort("a") is None
    assert lp.s.abort("b") is b                                      # still waiting
    assert "a" not in lp.cm and lp.cm.free_pages() == 50
    assert not lp.s.has_work()


def test_max_model_len_and_zero_tokens():
    lp = Loop(num_pages=50, max_batch_tokens=64, max_model_len=12)
    a, z, big = req("a", 8, max_tokens=100), req("z", 3, max_tokens=0), req("big", 12, max_tokens=5)
    for r in (a, z, big):
        lp.s.add(r)
    lp.run()
    assert a.finish_reason == "length" and a.total_len == 12
    assert z.finish_reason == "length" and z.output == []
    assert big.finish_reason == "too_long"


def test_same_arrivals_same_schedule():
    def trace():
        lp = Loop(num_pages=12, page_size=4, max_seqs=3, max_batch_tokens=10)
        for i in range(6):
            lp.s.add(req(i, 3 + 2 * i, max_tokens=7))
        lp.run()
        return [[(s.request.request_id, s.start, len(s.tokens), s.sample) for s in h.batch] for h in lp.history]
    assert trace() == trace()


def test_stop_sequences_end_the_stream_and_are_taken_back():
    """A sequence of token ids that ends the output stream stops the request the moment its last token is drawn
    (crates/scheduler/src/stop.rs:1-13); none of its tokens stays in the output.  A sequence that only begins
    to match, or matches across the prompt's end, does nothing."""
    free = Loop(64, max_seqs=2, max_batch_tokens=64)
    unstopped = req("a", 6, max_tokens=12, ignore_eos=True)
    free.s.add(unstopped)
    free.run()
    whole = unstopped.output
    assert len(whole) == 12 and len(set(whole)) == 12

    def run(seqs, **kw):
        loop = Loop(64, max_seqs=2, max_batch_tokens=64)
        r = req("a", 6, max_tokens=12, ignore_eos=True, stop_sequences=seqs, **kw)
        loop.s.add(r)
        loop.run()
        loop.cm.check()
        assert loop.cm.free_pages() == loop.cm.total_pages()
        return r

    r = run((tuple(whole[4:7]),))                      # tokens 4, 5, 6 of the free run: stops there, all three gone
    assert r.finish_reason == "stop" and r.output == whole[:4]
    r = run((tuple(whole[0:1]),))                      # a sequence of one token acts like a stop token
    assert r.finish_reason == "stop" and r.output == []
    r = run(((whole[5], whole[4]), (), (whole[3], 999)))   # wrong order, empty, a beginning only: no stop
    assert r.finish_reason == "length" and r.output == whole
    r = run(((6, whole[0]),))                          # would match only together with the prompt's last token
    assert r.finish_reason == "length" and r.output == whole
    r = run((tuple(whole[5:7]), tuple(whole[3:7])))    # two sequences end at the same token: the longer one is taken back
    assert r.finish_reason == "stop" and r.output == whole[:3]
    with pytest.raises(ValueError, match="stop_sequences"):
        run(((1, -2),))
