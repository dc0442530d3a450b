"""Generation through the entry point: greedy against the plain implementation, long
decoding, the sampler's options, preemption on the device, the command line."""
from __future__ import annotations

import os
import subprocess
import sys

import pytest
import torch

import plain_qwen3 as plain
import tiny

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model_dirs(tmp_path_factory):
    return {w: tiny.make_model_dir(str(tmp_path_factory.mktemp(f"gen{w}")), w, torch.float32) for w in ("A", "B")}


def plain_greedy_teacher(cfg, w, prompt, n):
    return plain.greedy(cfg, w, prompt, n)


@pytest.mark.parametrize("which", ["A", "B"])
def test_greedy_matches_plain_float32(model_dirs, which):
    from reinfer_b200 import LLM, SamplingParams
    cfg, w = plain.read_model(model_dirs[which])
    seqs = tiny.sequences(which, lengths=[5, 17, 33] if which == "A" else [1, 9, 24, 50])
    llm = LLM(model_dirs[which], dtype="float32", page_size=tiny.TINY[which][2], num_pages=64, max_num_seqs=4,
              max_batch_tokens=16, max_chunk=7)
    outs = llm.generate(list(seqs.values()), SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    for o, p in zip(outs, seqs.values()):
        assert o.token_ids == plain.greedy(cfg, w, p, 8) and o.finish_reason == "length"
    assert llm.engine.cache.free_pages() == 64


def test_greedy_bfloat16_follows_plain_teacher_forced(model_dirs, tmp_path):
    """bfloat16 may pick another token where two logits are close; wherever it picks, the plain
    logits of ITS sequence must call that token best or nearly so."""
    from reinfer_b200 import LLM, SamplingParams
    d = tiny.make_model_dir(str(tmp_path / "b16"), "B", torch.bfloat16)
    cfg, w = plain.read_model(d)
    prompt = tiny.sequences("B", lengths=[24])["r0"]
    llm = LLM(d, dtype="bfloat16", page_size=8, num_pages=64, max_num_seqs=2, max_batch_tokens=64)
    out = llm.generate(prompt, SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True))[0].token_ids
    logits = plain.forward(cfg, w, prompt + out)
    for i, tok in enumerate(out):
        row = logits[len(prompt) - 1 + i]
        assert row[tok] >= row.max() - 3e-2 * row.abs().max()


def test_long_decoding_float32(model_dirs):
    """One request decoded over many pages, every logit row compared at the end."""
    from reinfer_b200.engine import Engine, StepEntry
    which = "A"
    cfg, w = plain.read_model(model_dirs[which])
    seq = tiny.sequences(which, lengths=[300], seed=21)["r0"]
    e = Engine.from_model_dir(model_dirs[which], dtype="float32", page_size=16, max_tokens=320, max_num_seqs=1)
    rows = [e.step([StepEntry("x", seq[:4], [0, 1, 2, 3])])]
    for t in seq[4:]:
        rows.append(e.step([StepEntry("x", [t], [0])]))
    got = torch.cat(rows).double().cpu()
    ref = plain.forward(cfg, w, seq)
    assert (got - ref).abs().max().item() <= 1e-4 * ref.abs().max().item()
    assert torch.equal(got.argmax(-1), ref.argmax(-1))


def test_first_tokens_of_a_sequence(model_dirs):
    """Positions 0, 1, 2: a single key, a one-token prompt, a first page hardly begun."""
    from reinfer_b200.engine import Engine, StepEntry
    for which in ("A", "B"):
        cfg, w = plain.read_model(model_dirs[which])
        for dtype, tol in (("float32", 1e-4), ("bfloat16", 3e-2)):
            e = Engine.from_model_dir(model_dirs[which], dtype=dtype, page_size=tiny.TINY[which][2], max_tokens=64,
                                      max_num_seqs=2)
            seq = [7, 3, 250]
            ref = plain.forward(cfg, w, seq)
            got = torch.cat([e.step([StepEntry("x", [t], [0])]) for t in seq]).double().cpu()
            assert (got - ref).abs().max().item() <= tol * ref.abs().max().item()
            one = e.step([StepEntry("y", [7], [0])]).double().cpu()
            assert (one[0] - ref[0]).abs().max().item() <= tol * ref.abs().max().item()


def test_sampler_options(model_dirs):
    from reinfer_b200.sampling import Sampler, SamplingParams
    torch.manual_seed(0)
    V = 1000
    logits = torch.randn(4, V, device="cuda") * 2
    logits[1, 17] = float("nan"); logits[2, :] = float("-inf")
    s = Sampler(V, 8, "cuda")
    greedy = s.sample(logits, [SamplingParams()] * 4, [1] * 4, [0] * 4)
    assert greedy[0] == int(logits[0].argmax()) and greedy[2] == -1
    assert greedy[1] == int(torch.nan_to_num(logits[1], nan=-1e30).argmax())
    tie = torch.zeros(1, V, device="cuda"); tie[0, 5] = tie[0, 900] = 3.0
    assert s.sample(tie, [SamplingParams()], [0], [0]) == [5]                       # first maximum
    # same (seed, step) -> same token; rows do not influence each other
    p = SamplingParams(temperature=0.8, seed=3)
    a = s.sample(logits[:1], [p], [3], [4])
    b = s.sample(torch.cat([logits[3:4], logits[:1]]), [p, p], [9, 3], [0, 4])
    assert a[0] == b[1]
    # top_k: only the k largest are ever drawn; top_p / min_p: only the head of the distribution
    row = logits[0:1]
    top5 = set(torch.topk(row[0], 5).indices.tolist())
    draws = {s.sample(row, [SamplingParams(temperature=1.5, top_k=5)], [11], [i])[0] for i in range(200)}
    assert draws <= top5 and len(draws) >= 3
    pr = torch.softmax(row[0] / 1.0, 0)
    srt = torch.sort(pr, descending=True)
    n_keep = int((torch.cumsum(srt.values, 0) < 0.5).sum()) + 1
    nucleus = set(srt.indices[:n_keep].tolist())
    draws = {s.sample(row, [SamplingParams(temperature=1.0, top_p=0.5)], [12], [i])[0] for i in range(200)}
    assert draws <= nucleus and len(draws) >= 2
    keep = set((pr >= pr.max() * 0.3).nonzero().flatten().tolist())
    draws = {s.sample(row, [SamplingParams(temperature=1.0, min_p=0.3)], [13], [i])[0] for i in range(100)}
    assert draws <= keep
    # frequencies follow softmax(logits / T)
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0] + [-30.0] * (V - 4)], device="cuda")
    n = 4000
    counts = torch.zeros(4)
    for i in range(0, n, 8):
        for t in s.sample(small.expand(8, V).contiguous(), [SamplingParams(temperature=1.0)] * 8, [21] * 8, list(range(i, i + 8))):
            counts[t] += 1
    want = torch.softmax(torch.tensor([2.0, 1.0, 0.0, -1.0]), 0)
    assert (counts / n - want).abs().max().item() < 0.03
    # repetition penalty moves the choice away from a repeated best token
    rep = torch.zeros(1, V, device="cuda"); rep[0, 7] = 2.0; rep[0, 8] = 1.9
    assert s.sample(rep, [SamplingParams(repeat_penalty=1.5)], [0], [0], [[7, 7, 3]]) == [8]
    assert s.sample(rep, [SamplingParams(presence_penalty=0.5)], [0], [0], [[7]]) == [8]
    assert s.sample(rep, [SamplingParams(repeat_penalty=1.5)], [0], [0], [[3, 4]]) == [7]
    # logit_bias is added before everything else: it can promote a token, remove one, and comes before the penalties
    assert s.sample(rep, [SamplingParams(logit_bias=((500, 10.0),))], [0], [0]) == [500]
    assert s.sample(rep, [SamplingParams(logit_bias=((7, -5.0), (900, 0.5)))], [0], [0]) == [8]
    assert s.sample(rep, [SamplingParams(logit_bias=((8, 0.2),), repeat_penalty=1.5)], [0], [0], [[8]]) == [7]   # (1.9+0.2)/1.5 < 2
    two = s.sample(rep.expand(2, V).contiguous(), [SamplingParams(logit_bias=((9, 5.0),)), SamplingParams()], [0, 0], [0, 0])
    assert two == [9, 7]                                                               # a row's bias is its own
    draws = {s.sample(rep, [SamplingParams(temperature=1.0, logit_bias=((3, 50.0),))], [5], [i])[0] for i in range(20)}
    assert draws == {3}
    with pytest.raises(ValueError):
        SamplingParams(logit_bias=((1, 0.5), (1, 0.7))).validate()


def test_temperature_generation_is_seeded_and_batch_independent(model_dirs):
    from reinfer_b200 import LLM, SamplingParams
    which = "B"
    seqs = list(tiny.sequences(which, lengths=[9, 24, 50]).values())
    sp = SamplingParams(temperature=0.8, seed=3, max_tokens=10, ignore_eos=True)

    def run(prompts, **kw):
        llm = LLM(model_dirs[which], dtype="float32", page_size=8, num_pages=64, max_num_seqs=4, **kw)
        return [o.token_ids for o in llm.generate(prompts, sp)]
    together = run(seqs, max_batch_tokens=16, max_chunk=7)
    alone = [run([p], max_batch_tokens=64)[0] for p in seqs]
    assert together == alone
    assert together == run(seqs, max_batch_tokens=16, max_chunk=7)
    assert len({tuple(t) for t in together}) == 3


def test_preemption_on_the_device_keeps_outputs(model_dirs):
    """A pool too small for three requests at once: the newest is preempted, recomputes prompt + output when it
    returns and goes on.  The tokens are the plain implementation's, as in a run that never preempted."""
    from reinfer_b200 import LLM, SamplingParams
    which = "A"
    cfg, w = plain.read_model(model_dirs[which])
    seqs = list(tiny.sequences(which, lengths=[20, 25, 30]).values())
    sp = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
    want = [plain.greedy(cfg, w, p, 40) for p in seqs]
    calm = LLM(model_dirs[which], dtype="float32", page_size=16, num_pages=64, max_num_seqs=4, max_batch_tokens=32)
    assert [o.token_ids for o in calm.generate(seqs, sp)] == want
    tight = LLM(model_dirs[which], dtype="float32", page_size=16, num_pages=9, max_num_seqs=4, max_batch_tokens=32)
    outs = tight.generate(seqs, sp)
    assert tight.last_stats["preemptions"] > 0 and sum(o.preemptions for o in outs) > 0
    assert [o.token_ids for o in outs] == want
    assert tight.engine.cache.free_pages() == 9
    tight.engine.cache.check()


def test_preemption_in_bfloat16_follows_plain_teacher_forced(tmp_path):
    """The same squeeze in bfloat16: a preempted request's recomputed cache must carry it on as before.  Wherever
    bfloat16 picks a token, the plain logits of ITS sequence call that token best or nearly so, before and after
    the preemption; and a run that never preempts picks the same tokens."""
    from reinfer_b200 import LLM, SamplingParams
    d = tiny.make_model_dir(str(tmp_path / "a16"), "A", torch.bfloat16)
    cfg, w = plain.read_model(d)
    seqs = list(tiny.sequences("A", lengths=[20, 25, 30]).values())
    sp = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
    tight = LLM(d, dtype="bfloat16", page_size=16, num_pages=9, max_num_seqs=4, max_batch_tokens=32)
    outs = tight.generate(seqs, sp)
    assert sum(o.preemptions for o in outs) > 0
    for o, prompt in zip(outs, seqs):
        assert len(o.token_ids) == 40
        logits = plain.forward(cfg, w, prompt + o.token_ids)
        for i, tok in enumerate(o.token_ids):
            row = logits[len(prompt) - 1 + i]
            assert row[tok] >= row.max() - 3e-2 * row.abs().max(), f"token {i} after {o.preemptions} preemptions"
    tight.engine.cache.check()
    assert tight.engine.cache.free_pages() == 9


def test_a_step_that_fails_leaves_the_cache_as_it_was(tmp_path, monkeypatch):
    """A kernel wrapper raises in the middle of a step, after pages were reserved and a new request got its slot:
    the step's admissions and reservations are undone, the requests are as before, and the same step then runs
    and gives the logits of an engine that never failed."""
    from reinfer_b200 import ops
    from reinfer_b200.engine import Engine, StepEntry
    d = tiny.make_model_dir(str(tmp_path / "b16"), "B", torch.bfloat16)
    seqs = tiny.sequences("B", lengths=[40, 21])
    a, b = seqs["r0"], seqs["r1"]

    def fresh():
        e = Engine.from_model_dir(d, dtype="bfloat16", page_size=8, num_pages=12, max_num_seqs=2)
        e.step([StepEntry("a", a[:19], [18])])
        return e
    entries = [StepEntry("a", a[19:35], [15]), StepEntry("b", b[:13], [0, 12])]
    want = fresh().step(entries).clone()
    e = fresh()
    before = (e.cache.length("a"), list(e.cache.table("a", 0)), e.cache.slot("a"), e.cache.free_pages(), e.cache.free_slots())
    calls = {"n": 0}
    real = ops.attention

    def failing(*args, **kw):
        calls["n"] += 1
        if calls["n"] == 2:                             # in the second layer: the first has stored its keys by then
            raise ops.KernelError("injected")
        return real(*args, **kw)
    monkeypatch.setattr(ops, "attention", failing)
    with pytest.raises(ops.KernelError, match="injected"):
        e.step(entries)
    monkeypatch.setattr(ops, "attention", real)
    e.cache.check()
    assert "b" not in e.cache
    assert (e.cache.length("a"), list(e.cache.table("a", 0)), e.cache.slot("a"), e.cache.free_pages(), e.cache.free_slots()) == before
    got = e.step(entries)
    assert torch.equal(got, want)
    # a decode step (replayed from a captured graph) that fails while it is being built: the same
    one = [StepEntry("a", [a[35]], [0]), StepEntry("b", [b[13]], [0])]
    before = (e.cache.length("a"), len(e.cache.table("a", 0)), e.cache.length("b"), e.cache.free_pages())
    calls["n"] = 0
    monkeypatch.setattr(ops, "attention", failing)
    with pytest.raises(ops.KernelError, match="injected"):
        e.step(one)
    monkeypatch.setattr(ops, "attention", real)
    e.cache.check()
    assert (e.cache.length("a"), len(e.cache.table("a", 0)), e.cache.length("b"), e.cache.free_pages()) == before
    ref = fresh()
    ref.step(entries)
    assert torch.equal(e.step(one), ref.step(one))


def test_a_wait_that_runs_out_reaches_the_engine(model_dirs):
    """The kernels bound every wait; one that gives up sets a word that the engine reads.  Here the self-test
    kernel waits a millisecond for an arrival that never comes (no product kernel is made to fail): the word
    names it, `Engine.step` and `LLM.step` refuse to go on, the requests of the failed step give back their
    pages, and after `clear_status` the library and the engine work as before."""
    from reinfer_b200 import LLM, SamplingParams, ops
    from reinfer_b200.engine import Engine, KernelWaitTimeout, StepEntry
    e = Engine.from_model_dir(model_dirs["A"], dtype="float32", page_size=16, num_pages=8, max_num_seqs=2)
    first = e.step([StepEntry("x", [1, 2, 3], [2])]).clone()
    assert ops.status_word() == 0
    try:
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.test_bounded_wait(1_000_000, flag)
        torch.cuda.synchronize()
        assert int(flag.item()) == 1
        code = ops.status_word()
        assert code == (4 << 16) | (1 << 8) | 77
        assert "self-test" in ops.describe_status(code)
        with pytest.raises(KernelWaitTimeout, match="bounded wait gave up"):
            e.step([StepEntry("x", [4], [0])])
        assert e.cache.length("x") == 3                  # nothing was launched, nothing changed
        llm = LLM(engine=e, max_batch_tokens=16)
        rid = llm.add_request([5, 6, 7], SamplingParams(max_tokens=3, ignore_eos=True))
        with pytest.raises(KernelWaitTimeout):
            llm.step()
        assert llm.requests[rid].finish_reason == "error" and not llm.has_work()
        e.cache.check()
    finally:
        assert ops.clear_status() in (0, (4 << 16) | (1 << 8) | 77)
    assert ops.status_word() == 0 and ops.kernel_error() == 0
    a = torch.randn(5, 64, device="cuda").bfloat16()
    w = torch.randn(24, 64, device="cuda").bfloat16()
    c = torch.empty(5, 24, device="cuda")
    ops.gemm_bf16(a, w, c)
    assert (c - a.float() @ w.float().t()).abs().max().item() < 1e-2 * c.abs().max().item()
    again = e.step([StepEntry("y", [1, 2, 3], [2])])
    assert torch.equal(again, first)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_requests_leave_a_decoding_batch_at_different_steps(tmp_path, dtype):
    """Distinct token limits, a stop token, a stop sequence and the end-of-sequence id of config.json, all
    honoured: the requests leave the batch one after another while the others go on.  Decode steps are replayed
    from graphs and launched ahead of the reading of the step before; a request that ends by a token the host
    could not foresee has a row in the step already running, which is dropped.  The outputs are the plain
    implementation's greedy tokens cut at the same places (bfloat16: checked token by token against the plain
    logits of its own sequence)."""
    import json
    from reinfer_b200 import LLM, SamplingParams
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    d = tiny.make_model_dir(str(tmp_path / "m"), "B", store)
    cfg, w = plain.read_model(d)
    prompts = list(tiny.sequences("B", lengths=[9, 24, 5, 17, 30, 12], seed=13).values())
    free_run = [plain.greedy(cfg, w, p, 24) for p in prompts]
    # the end-of-sequence id: what request 0 draws as its 11th token; request 1 stops on its own 7th token;
    # request 2 on the sequence of its 13th and 14th
    eos = free_run[0][10]
    raw = json.load(open(f"{d}/config.json"))
    raw["eos_token_id"] = eos
    json.dump(raw, open(f"{d}/config.json", "w"))
    params = [SamplingParams(max_tokens=24), SamplingParams(max_tokens=24, stop_token_ids=(free_run[1][6],)),
              SamplingParams(max_tokens=24, stop_sequences=((free_run[2][12], free_run[2][13]),)),
              SamplingParams(max_tokens=5), SamplingParams(max_tokens=16, ignore_eos=True), SamplingParams(max_tokens=21)]

    def cut(tokens, p):
        out = []
        for t in tokens[:p.max_tokens]:
            if t in p.stop_token_ids:
                return out, "stop"
            if any(len(q) and list(q) == (out + [t])[-len(q):] for q in p.stop_sequences):
                return out[:len(out) - (max(len(q) for q in p.stop_sequences if list(q) == (out + [t])[-len(q):]) - 1)], "stop"
            if t == eos and not p.ignore_eos:
                return out, "eos"
            out.append(t)
        return out, "length"
    llm = LLM(d, dtype=dtype, page_size=8, num_pages=64, max_num_seqs=8, max_batch_tokens=64)
    assert llm.eos == (eos,)
    outs = llm.generate(prompts, params)
    assert llm.engine.graph_replays > 0 and llm.steps_launched_ahead > 0 and llm.ahead_rows_dropped > 0
    assert llm.engine.cache.free_pages() == 64 and not llm.has_work()
    llm.engine.cache.check()
    if dtype == "float32":
        for o, free, p in zip(outs, free_run, params):
            want, why = cut(free, p)
            assert (o.token_ids, o.finish_reason) == (want, why), f"request {o.request_id}"
        assert len({len(o.token_ids) for o in outs}) >= 4            # they did leave at different steps
    else:
        for o, prompt, p in zip(outs, prompts, params):
            logits = plain.forward(cfg, w, prompt + o.token_ids)
            for i, tok in enumerate(o.token_ids):
                row = logits[len(prompt) - 1 + i]
                assert row[tok] >= row.max() - 3e-2 * row.abs().max()
            assert len(o.token_ids) <= p.max_tokens and o.finish_reason in ("stop", "eos", "length")
            assert (o.finish_reason == "length") == (len(o.token_ids) == p.max_tokens)


def test_penalties_through_the_slots_follow_the_host_driven_sampler(model_dirs):
    """Generation with a repetition and a presence penalty, a logit bias and a temperature: the sampler works from
    the requests' slots on the device (record, ring of drawn tokens, draw count kept by the kernel itself).  The
    same tokens come out when every step's logits are sampled by the host-driven entry point with the history and
    step count that the host keeps - and when the pool is so small that requests are preempted and return."""
    from reinfer_b200 import LLM, SamplingParams
    from reinfer_b200.engine import Engine, StepEntry
    from reinfer_b200.sampling import Sampler
    which = "A"
    prompts = list(tiny.sequences(which, lengths=[6, 11, 19], seed=17).values())
    sps = [SamplingParams(temperature=0.0, repeat_penalty=1.4, repeat_last_n=5, max_tokens=30, ignore_eos=True),
           SamplingParams(temperature=0.9, seed=5, presence_penalty=0.7, frequency_penalty=0.2, max_tokens=30, ignore_eos=True),
           SamplingParams(temperature=0.7, seed=6, top_k=20, logit_bias=((3, 2.0), (9, -4.0)), repeat_penalty=1.2,
                          max_tokens=30, ignore_eos=True)]
    llm = LLM(model_dirs[which], dtype="float32", page_size=16, num_pages=64, max_num_seqs=4, max_batch_tokens=32)
    got = [o.token_ids for o in llm.generate(prompts, sps)]
    tight = LLM(model_dirs[which], dtype="float32", page_size=16, num_pages=6, max_num_seqs=4, max_batch_tokens=32)
    outs = tight.generate(prompts, sps)
    assert sum(o.preemptions for o in outs) > 0
    assert [o.token_ids for o in outs] == got
    # the reference run: one request at a time, logits from the step function, the host-driven sampler
    e = Engine.from_model_dir(model_dirs[which], dtype="float32", page_size=16, num_pages=64, max_num_seqs=1)
    s = Sampler(e.vocab_size, 1, "cuda")
    for prompt, sp, toks in zip(prompts, sps, got):
        out = []
        logits = e.step([StepEntry("r", prompt, [len(prompt) - 1])])
        for n in range(sp.max_tokens):
            t = s.sample(logits, [sp], [sp.seed or 0], [n], [out[-sp.repeat_last_n:]])[0]
            out.append(t)
            logits = e.step([StepEntry("r", [t], [0])])
        e.finish("r")
        if sp.seed is not None or sp.temperature == 0.0:
            assert out == toks


def test_step_profile_flag_changes_no_token(model_dirs, monkeypatch):
    """REINFER_B200_STEP_PROFILE runs some steps eagerly with events behind every launch: the same tokens, and a
    report by kernel family."""
    from reinfer_b200.engine.llm import LLM
    from reinfer_b200.sampling import SamplingParams
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    prompts = [t[:9] for t in list(tiny.sequences("A").values())[:2]]
    plain_run = LLM(model_dirs["A"], dtype="bfloat16", max_num_seqs=4, page_size=16, num_pages=32).generate(prompts, sp)
    monkeypatch.setenv("REINFER_B200_STEP_PROFILE", "decode:3")
    llm = LLM(model_dirs["A"], dtype="bfloat16", max_num_seqs=4, page_size=16, num_pages=32)
    outs = llm.generate(prompts, sp)
    assert [o.token_ids for o in outs] == [o.token_ids for o in plain_run]
    report = llm.profile_report()
    assert len(llm._profile_runs) >= 3 and report and "decode" in report[0]
    assert any(line.startswith("sample_slots") for line in report) and any(line.startswith("total") for line in report)


def test_guard_pages_tell_of_a_store_beside_the_pool(model_dirs):
    """The pages around a layer's own hold a pattern; a store to page -1 (made here by hand) is reported with the
    layer's name, and nothing else is."""
    from reinfer_b200.engine import Engine, EngineError, StepEntry
    engine = Engine.from_model_dir(model_dirs["A"], dtype="bfloat16", max_tokens=256, max_num_seqs=2)
    engine.step([StepEntry("a", list(range(3, 40)), [36])])
    engine.check_guards()
    name, kv = next(iter(engine.storage.layer_kv.items()))
    page_elems = kv[0].numel()
    flat = kv.reshape(-1)
    torch.as_strided(flat, (4,), (1,), flat.storage_offset() - page_elems + 5).fill_(1.0)     # four elements of page -1
    with pytest.raises(EngineError, match=f"{name}: before"):
        engine.check_guards()
    assert engine.storage.check_guards() == [f"{name}: before"]


def test_out_of_vocabulary_token_is_refused(model_dirs):
    from reinfer_b200.engine import EmbeddingOov, Engine, StepEntry
    e = Engine.from_model_dir(model_dirs["A"], dtype="float32", max_tokens=64, max_num_seqs=1)
    with pytest.raises(EmbeddingOov):
        e.step([StepEntry("x", [1, 256], [1])])
    assert "x" not in e.cache


def test_command_line(model_dirs):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, w = plain.read_model(model_dirs["A"])
    prompt = [4, 8, 15, 16, 23, 42]
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "reinfer"), "run", model_dirs["A"], "-n", "5", "-t", "0",
                        "--dtype", "float32", "--perf"] + [str(t) for t in prompt], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = p.stdout.strip().splitlines()
    assert [int(t) for t in lines[0].split()] == plain.greedy(cfg, w, prompt, 5)
    assert lines[1].startswith("PERF ") and "tpot_ms=" in lines[1]
