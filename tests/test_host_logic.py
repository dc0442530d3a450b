"""Host-side decisions of the kernel layer that need no GPU: what the streaming kernels learn about the order
of the weights, how many CTAs share a request's keys in decode attention, and the sampler's parameter checks."""
from __future__ import annotations

import pytest


def test_stream_chain_learns_the_order_of_a_pass_and_forgets_a_changed_one():
    from reinfer_b200.ops import StreamChain
    c = StreamChain()
    a, b, d = (0x1000, 64), (0x2000, 128), (0x3000, 32)
    assert c.step(*a) is None                       # outside a pass: nothing is noted
    c.begin()
    assert c.step(*a) is None and c.step(*b) is None and c.step(*d) is None     # the first pass only writes down
    c.end()
    c.begin()
    assert c.step(*a) == b and c.step(*b) == d and c.step(*d) == a              # after the last range comes the first
    c.end()
    # a pass that streams something else at a place gets no hint there, and the pass after it learns the new order
    c.begin()
    assert c.step(*a) == b
    assert c.step(0x9000, 8) is None
    assert c.step(*d) == a                          # places are compared one by one: the third still matches
    c.end()
    c.begin()
    assert c.step(*a) == (0x9000, 8) and c.step(0x9000, 8) == d and c.step(*d) == a
    c.end()
    # a pass that did not complete (no end()) leaves what is known as it was
    c.begin()
    c.step(*b)
    c.live = False
    c.begin()
    assert c.step(*a) == (0x9000, 8)
    # markers (zero bytes) take a place in the order but are never offered for prefetching
    m = StreamChain()
    for _ in range(2):
        m.begin()
        r1 = m.step(*a)
        r2 = m.step(0x7777, 0)
        r3 = m.step(*b)
        m.end()
    assert r1 is None and r2 == b and r3 == a
    # unaligned ranges are not offered either
    u = StreamChain()
    for _ in range(2):
        u.begin()
        r = u.step(*a)
        u.step(0x2008, 64)
        u.end()
    assert r is None


def test_decode_splits_model():
    from functools import partial
    from reinfer_b200 import ops
    # what the device says about clusters of more than 8 CTAs is an argument here: all slots, or none
    decode_splits = partial(ops.decode_splits, cluster_slots=lambda n: ops.DECODE_SLOTS)
    portable_only = partial(ops.decode_splits, cluster_slots=lambda n: 0)
    # many (request, kv head) pairs: one CTA each streams at the memory bandwidth, splitting only adds fill and drain
    assert decode_splits(64 * 8, 64) == 1
    assert decode_splits(32 * 8, 64) == 1
    # a few more pairs than the device holds at once: unsplit, the CTAs of the part-filled last wave would walk their
    # tiles alone; three splits make the waves short (measured at 40 and 48 requests), but not where the last wave
    # is well filled anyway (56, 64)
    assert decode_splits(40 * 8, 64) in (3, 4)             # measured: 3 and 4 alike, a tenth faster than 1
    assert decode_splits(48 * 8, 64) in (2, 3)             # measured: 3, then 2; 4 no better than 1
    assert decode_splits(56 * 8, 64) == 1
    assert decode_splits(37 * 8, 64) == 1                  # exactly the places there are
    # few pairs: splits until enough CTAs stream; they stay inside a cluster while all are resident at once
    assert decode_splits(16 * 8, 64) == 2
    assert decode_splits(8 * 8, 64) == 4
    assert 2 <= decode_splits(4 * 8, 64) <= 8
    # one request: as many splits as the largest cluster holds; where the device allows only portable clusters,
    # the largest portable cluster or more splits than that, merged by a kernel
    assert decode_splits(8, 64) == 16
    assert portable_only(8, 64) >= 8 and portable_only(8, 64) != 16
    # never more splits than tiles, never fewer than one
    for ctas in (1, 8, 64, 512, 4096):
        for tiles in (1, 2, 3, 16, 64, 512, 2048):
            for f in (decode_splits, portable_only):
                n = f(ctas, tiles)
                assert 1 <= n <= max(1, min(64, tiles))
    assert decode_splits(8, 1) == 1
    # requests of unequal lengths (32 of them, the longest 67 tiles, 36 on average): one CTA per pair would last as
    # long as the longest request; two splits halve that although the CTAs no longer fit the device at once
    assert decode_splits(32 * 8, 67) == 1
    assert decode_splits(32 * 8, 67, total_tiles=32 * 8 * 36) == 2
    # wider heads: the same decisions at the same number of bytes
    assert decode_splits(64 * 8, 64, head_dim=256) == 1


def test_sampling_params_checks():
    from reinfer_b200.sampling import SamplingParams
    SamplingParams(logit_bias=((3, 1.5), (9, -2.0))).validate()
    with pytest.raises(ValueError):
        SamplingParams(logit_bias=((3, 1.0), (3, 2.0))).validate()
    with pytest.raises(ValueError):
        SamplingParams(logit_bias=((-1, 1.0),)).validate()
    with pytest.raises(ValueError):
        SamplingParams(logit_bias=tuple((i, 0.1) for i in range(1025))).validate()
    with pytest.raises(ValueError):
        SamplingParams(repeat_last_n=65).validate()
    with pytest.raises(ValueError):
        SamplingParams(max_tokens=-1).validate()


# ---------------------------------------------------------------- the command line's host side
def test_model_folder_resolution(tmp_path, monkeypatch):
    """A local folder wins; a bare name is looked up under $REINFER_MODEL_DIR (bin/reinfer/src/main.rs:540-558)."""
    from reinfer_b200.cli import resolve_model_dir
    local = tmp_path / "here"
    local.mkdir()
    assert resolve_model_dir(str(local)) == str(local)
    root = tmp_path / "models"
    (root / "org" / "tiny").mkdir(parents=True)
    (root / "org" / "tiny" / "config.json").write_text("{}")
    monkeypatch.setenv("REINFER_MODEL_DIR", str(root))
    assert resolve_model_dir("org/tiny") == str(root / "org" / "tiny")
    with pytest.raises(FileNotFoundError, match="REINFER_MODEL_DIR"):
        resolve_model_dir("org/absent")


def test_command_line_refuses_other_backends_and_missing_models(tmp_path, capsys, monkeypatch):
    from reinfer_b200.cli import main
    monkeypatch.setenv("REINFER_MODEL_DIR", str(tmp_path))
    assert main(["run", "nobody/nothing", "1", "2"]) == 2
    assert "model not found locally" in capsys.readouterr().err
    (tmp_path / "m").mkdir()
    assert main(["run", str(tmp_path / "m"), "--backend", "cpu", "1", "2"]) == 2
    assert "cuda" in capsys.readouterr().err


# ---------------------------------------------------------------- bench.py's answers that need no GPU
def test_bench_refuses_more_than_one_gpu_and_names_the_reference_arm():
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--gpus", "2"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 2
    said = (p.stdout + p.stderr).strip().splitlines()
    assert len(said) == 1 and "one GPU" in said[0]
    p = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                        "--warmup", "1"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0
    rec = json.loads(p.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and rec["unavailable"]


def test_penalty_window_holds_sampled_tokens_only():
    """What the repeat / frequency / presence penalties look at: the last `repeat_last_n` tokens the request has
    drawn - none of its prompt - laid out as the ring that the kernel goes on writing (draw n at n mod window)."""
    from reinfer_b200.sampling.sampler import history_ring
    ring, valid = history_ring([], 64)                       # the first token: nothing to penalise yet
    assert valid == 0 and ring.shape == (64,)
    ring, valid = history_ring([7, 8, 9], 64)                # fewer draws than the window
    assert valid == 3 and ring[:3].tolist() == [7, 8, 9]
    drawn = list(range(100, 110))                            # more draws than the window: the last 4, each at n mod 4
    ring, valid = history_ring(drawn, 4)
    assert valid == 4 and sorted(ring.tolist()) == [106, 107, 108, 109]
    assert all(ring[n % 4] == drawn[n] for n in range(6, 10))
    # a request that was preempted keeps its output and returns with the same ring (the prompt never enters)
    again, valid2 = history_ring(list(drawn), 4)
    assert valid2 == valid and again.tolist() == ring.tolist()
    assert history_ring([1, 2, 3], 0)[1] == 0                # penalties off: no window


def test_a_failed_step_ends_its_requests_and_stops_the_loop():
    """The entry point's answer to an engine error (a kernel whose bounded wait gave up sets a word that
    `Engine.step` raises on): nothing of the step is recorded, its requests end with "error" and give back
    what they hold, and the error goes on to the caller."""
    from reinfer_b200.cache import CacheManager
    from reinfer_b200.engine.engine import KernelWaitTimeout
    from reinfer_b200.engine.scheduler import Request, Scheduler
    from reinfer_b200.parts.base import PagedKVSpec
    from reinfer_b200.sampling import SamplingParams
    cm = CacheManager({"l0": PagedKVSpec(2, 16)}, {}, 4, 16, 4)
    released = []

    def release(rid):
        released.append(rid)
        if rid in cm:
            cm.release(rid)
    s = Scheduler(cm, max_batch_tokens=32, release=release)
    a, b = Request("a", [1, 2, 3], SamplingParams(max_tokens=4)), Request("b", [4, 5], SamplingParams(max_tokens=4))
    s.add(a); s.add(b)
    out = s.schedule()
    for x in out.batch:                                      # what the engine does before it launches
        cm.admit(x.request.request_id)
        cm.reserve(x.request.request_id, len(x.tokens))
    try:
        raise KernelWaitTimeout("a bounded wait gave up")    # what Engine.step / check_status raise
    except KernelWaitTimeout:
        for x in out.batch:
            s.fail(x.request)
    assert a.finish_reason == b.finish_reason == "error" and not a.output and a.num_computed == 0
    assert sorted(released) == ["a", "b"] and not s.has_work()
    assert cm.free_pages() == cm.total_pages() and cm.free_slots() == 4
    cm.check()


# ---------------------------------------------------------------- a block's hand-overs, with stand-in parts (no device)

def test_prenorm_block_hands_sums_and_prepared_rows_on():
    """What the pre-norm arrangement passes between its parts, seen with stand-ins on the CPU: a part's return value
    (nothing, a sum still to be added, or rows that a product prepared for the norm that reads the residual next)
    reaches exactly that norm; the norm that a part may prepare for is named only while that part runs, and only if
    norm and reader both know the form; across blocks the model's loop names the next block's first norm."""
    import torch
    from reinfer_b200.parts.base import PreparedRows, RowScaled
    from reinfer_b200.parts.block import PreNormBlock

    log = []

    class Ctx:
        norm_ahead = None
        norm_after_block = None

    class NormStandIn:
        adds_partial_sums = True

        def __init__(self, name, scaled):
            self.name, self.leaves_row_scale = name, scaled
            if scaled:
                self.prepared_by = lambda ctx, a, w, residual: PreparedRows(self, torch.ones(2, 4), torch.ones(2, 1))

        def forward(self, ctx, x, out=None, delta=None, row_idx=None, scaled_ok=False):
            log.append((self.name, type(delta).__name__, scaled_ok))
            if isinstance(delta, PreparedRows):
                assert delta.norm is self and scaled_ok
                return RowScaled(delta.rows, delta.sumsq, 4, 1e-6)
            return x + (0 if delta is None else delta)

    class PartStandIn:
        def __init__(self, name, takes, result):
            self.name, self.takes_row_scaled, self.result = name, takes, result

        def forward(self, ctx, xn, residual, cache=None):
            ahead = ctx.norm_ahead
            log.append((self.name, type(xn).__name__, None if ahead is None else ahead.name))
            if self.result == "prepared" and ahead is not None:
                return ahead.prepared_by(ctx, None, None, residual)
            return torch.full((2, 4), 0.5) if self.result == "sum" else None

    x = torch.zeros(2, 4)
    # both sides know the form: the mixer is told of the ffn's norm, prepares its rows, the ffn gets them as RowScaled;
    # the ffn is told of the norm after the block (here: the next block's first norm) and hands its rows out
    n1, n2, nxt = NormStandIn("mixer_norm", True), NormStandIn("ffn_norm", True), NormStandIn("next", True)
    block = PreNormBlock({"mixer_norm": n1, "mixer": PartStandIn("mixer", True, "prepared"),
                          "ffn_norm": n2, "ffn": PartStandIn("ffn", True, "prepared")})
    ctx = Ctx()
    ctx.norm_after_block = nxt
    out = block.forward(ctx, x, None, None)
    assert isinstance(out, PreparedRows) and out.norm is nxt
    assert ctx.norm_ahead is None                                   # named only while the part runs
    assert log == [("mixer_norm", "NoneType", True), ("mixer", "Tensor", "ffn_norm"),
                   ("ffn_norm", "PreparedRows", True), ("ffn", "RowScaled", "next")]
    assert block.entry_norm() is n1
    # a reader that does not take rows without their factor: nobody is named, sums go the plain way
    log.clear()
    block = PreNormBlock({"mixer_norm": n1, "mixer": PartStandIn("mixer", False, "sum"),
                          "ffn_norm": n2, "ffn": PartStandIn("ffn", False, None)})
    ctx = Ctx()
    assert block.forward(ctx, x, None, torch.ones(2, 4)) is None
    assert log == [("mixer_norm", "Tensor", False), ("mixer", "Tensor", None),
                   ("ffn_norm", "Tensor", False), ("ffn", "Tensor", None)]
    assert block.entry_norm() is None
    # a norm that cannot have its rows prepared is never named, whatever its reader takes
    plain_norm = NormStandIn("plain", False)
    block = PreNormBlock({"mixer_norm": plain_norm, "mixer": PartStandIn("mixer", True, "prepared"),
                          "ffn_norm": plain_norm, "ffn": PartStandIn("ffn", True, "prepared")})
    log.clear()
    ctx = Ctx()
    ctx.norm_after_block = nxt
    out = block.forward(ctx, x, None, None)
    assert [e[2] for e in log if e[0] == "mixer"] == [None]          # the mixer was told of no norm
    assert isinstance(out, PreparedRows)                            # the ffn still prepares for the next block's norm
