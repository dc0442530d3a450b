"""The engine against the plain implementation, in 32-bit and in bfloat16, under every
way of cutting the work: whole, tail one by one, portions down to two tokens, mixed
batches over a pool so small that pages are used again."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import tiny

pytestmark = pytest.mark.gpu

# |engine - plain| <= TOL * max|plain logit| of the row
TOL = {"float32": 1e-4, "bfloat16": 3e-2}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for which in ("A", "B"):
        for store, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
            d = str(tmp_path_factory.mktemp(f"tiny{which}_{store}"))
            tiny.make_model_dir(d, which, dt)
            out[(which, store)] = d
    return out


_truth_cache = {}


def truth(model_dir, seqs):
    key = (model_dir, tuple((r, tuple(t)) for r, t in seqs.items()))
    if key not in _truth_cache:
        cfg, w = plain.read_model(model_dir)
        _truth_cache[key] = {r: plain.forward(cfg, w, t) for r, t in seqs.items()}
    return _truth_cache[key]


def run_steps(engine, steps, owners=None):
    """-> {(request, position): logits row (cpu float64)}"""
    from reinfer_b200.engine import StepEntry
    got = {}
    done = {}
    for entries, end in steps:
        logits = engine.step([StepEntry(r, t, w) for r, t, w in entries])
        if owners is not None:
            owners.look()
        row = 0
        for r, t, w in entries:
            base = done.get(r, 0)
            for k in w:
                got[(r, base + k)] = logits[row].double().cpu()
                row += 1
            done[r] = base + len(t)
        for r in end:
            engine.finish(r)
            done.pop(r, None)
        engine.cache.check()
    engine.check_guards()                       # no store reached a page beside a layer's own
    return got


def compare(got, want, tol):
    worst = 0.0
    for (r, p), row in got.items():
        ref = want[r][p]
        scale = ref.abs().max().item()
        err = (row - ref).abs().max().item() / scale
        worst = max(worst, err)
        assert err <= tol, f"request {r} position {p}: error {err:.3e} of the logit scale (limit {tol})"
        top2 = torch.topk(ref, 2).values
        if (top2[0] - top2[1]).item() > 2 * tol * scale:
            assert int(row.argmax()) == int(ref.argmax()), f"request {r} position {p}: other argmax"
    return worst


CUTS = {"whole": tiny.cut_whole, "tail": tiny.cut_tail_one_by_one, "portions": tiny.cut_portions,
        "mixed": tiny.cut_mixed}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B"])
@pytest.mark.parametrize("cut", list(CUTS))
def test_cuts_match_plain(models, which, dtype, cut):
    from reinfer_b200.engine import Engine
    model_dir = models[(which, "f32" if dtype == "float32" else "bf16")]
    seqs = tiny.sequences(which)
    steps = CUTS[cut](seqs)
    page = tiny.TINY[which][2]
    pool = tiny.pool_tokens_needed(steps, page)          # exactly the pages the steps need: not one to spare
    engine = Engine.from_model_dir(model_dir, dtype=dtype, page_size=page, max_tokens=pool, max_num_seqs=4)
    owners = tiny.PageOwners(engine.cache)
    got = run_steps(engine, steps, owners)
    assert len(got) == sum(len(t) for t in seqs.values())
    compare(got, truth(model_dir, seqs), TOL[dtype])
    assert engine.cache.free_pages() == engine.cache.total_pages()
    if cut == "mixed":
        # finished requests' pages went to later requests: at least half of the pool had a second owner
        assert 2 * len(owners.reused) >= engine.cache.total_pages(), (len(owners.reused), engine.cache.total_pages())


@pytest.mark.parametrize("which", ["A", "B"])
def test_float32_cuts_agree_bitwise(models, which):
    """The 32-bit kernels order their sums by position only, so every cut gives the same bits."""
    from reinfer_b200.engine import Engine
    model_dir = models[(which, "f32")]
    seqs = tiny.sequences(which)
    results = []
    for cut in CUTS.values():
        steps = cut(seqs)
        engine = Engine.from_model_dir(model_dir, dtype="float32", page_size=tiny.TINY[which][2],
                                       max_tokens=tiny.pool_tokens_needed(steps, tiny.TINY[which][2]), max_num_seqs=4)
        results.append(run_steps(engine, steps))
    for other in results[1:]:
        for key, row in results[0].items():
            assert torch.equal(row, other[key]), f"{key}: bits differ between cuts"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(models, tmp_path, dtype):
    """bin/trace_run end to end: protocol, files, pages used again."""
    which = "B"
    model_dir = models[(which, "f32" if dtype == "float32" else "bf16")]
    seqs = tiny.sequences(which)
    steps = tiny.cut_mixed(seqs, seed=11)
    lines = []
    for i, (entries, end) in enumerate(steps):
        lines.append(json.dumps({"step": i, "entries": [{"id": r, "tokens": t, "want": w} for r, t, w in entries],
                                 "end": end}))
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    extra = ["--page-size", "16"] if dtype == "float32" else []      # the default page (64 tokens) and a smaller one
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
                        "--out", str(out), "--max-tokens", str(tiny.pool_tokens_needed(steps))] + extra,
                       input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    want = truth(model_dir, seqs)
    vocab = tiny.TINY[which][0]["vocab_size"]
    done, got = {}, {}
    for i, (entries, end) in enumerate(steps):
        arr = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, vocab)
        row = 0
        for r, t, w in entries:
            for k in w:
                got[(r, done.get(r, 0) + k)] = torch.from_numpy(arr[row].astype(np.float64))
                row += 1
            done[r] = done.get(r, 0) + len(t)
        assert row == arr.shape[0]
    compare(got, want, TOL[dtype])


@pytest.mark.parametrize("store,dtype", [("f32", "bfloat16"), ("bf16", "float32")])
def test_storage_and_compute_dtype_may_differ(models, store, dtype):
    """A folder stored in 32 bits run in bfloat16 (its tensors stay 32-bit: the plain kernels take the
    products) and a folder stored in bfloat16 run in float32 (widened): both against the plain
    implementation of the stored values."""
    from reinfer_b200.engine import Engine
    which = "B"
    model_dir = models[(which, store)]
    seqs = tiny.sequences(which)
    steps = tiny.cut_mixed(seqs, seed=5)
    engine = Engine.from_model_dir(model_dir, dtype=dtype, page_size=8, max_tokens=tiny.pool_tokens_needed(steps, 8), max_num_seqs=4)
    if store == "f32":
        assert engine.model.layers[0].mixer.w_qkv.dtype == torch.float32
    got = run_steps(engine, steps)
    compare(got, truth(model_dir, seqs), TOL[dtype])


def test_a_decode_layer_is_five_launches_and_equals_the_separate_kernels(tmp_path, monkeypatch):
    """With heads of 128 and a width in tiles of 128 a decode step's layer runs as five launches (the norms, the
    residual sums and the per-head work ride in the products' reductions).  The count is asserted, so that a silent
    fall back to the separate kernels shows; and the logits equal, to rounding, those of the same step with the
    separate kernels (the switches that bring them back), which in turn follow the plain implementation."""
    from reinfer_b200 import ops
    from reinfer_b200.config import Qwen3Config
    from reinfer_b200.engine import Engine
    from reinfer_b200.weights import write_random_model
    layers = 3
    raw = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=layers, hidden_size=256, num_attention_heads=4,
               num_key_value_heads=2, head_dim=128, intermediate_size=384, vocab_size=1003, rope_theta=1e6,
               rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=1024)
    d = write_random_model(str(tmp_path / "m"), Qwen3Config.from_dict(raw), seed=3, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(8)
    seqs = {f"r{i}": torch.randint(0, 1003, (n,), generator=g).tolist() for i, n in enumerate((70, 9, 130))}
    names = list(seqs)
    steps = [([(r, seqs[r][:-4], [len(seqs[r]) - 5]) for r in names], [])]
    for k in range(4, 0, -1):
        steps.append(([(r, [seqs[r][-k]], [0]) for r in names], names if k == 1 else []))
    cfg, w = plain.read_model(d)
    want = {r: plain.forward(cfg, w, t, dtype=torch.float32).double() for r, t in seqs.items()}

    def run(product_norm, qkv_heads):
        monkeypatch.setattr(ops, "PRODUCT_NORM", product_norm)
        monkeypatch.setattr(ops, "QKV_HEADS", qkv_heads)
        engine = Engine.from_model_dir(d, dtype="bfloat16", page_size=16, max_tokens=3 * 192, max_num_seqs=4)
        got = run_steps(engine, steps)
        graphs = list(engine._graphs.values())
        assert graphs, "decode steps replay a graph"
        return got, graphs[0].n_launches

    fused, n_fused = run(True, True)
    apart, n_apart = run(False, False)
    # embedding, final norm, head - and the first layer's norm, which no product precedes; five a layer against eight
    assert n_fused == 4 + 5 * layers, n_fused
    assert n_apart == 3 + 8 * layers, n_apart
    compare(fused, want, TOL["bfloat16"])
    compare(apart, want, TOL["bfloat16"])
    for key in fused:
        a, b = fused[key].double(), apart[key].double()
        assert (a - b).abs().max().item() <= 2e-2 * max(b.abs().max().item(), 1.0)
    assert ops.kernel_error() == 0


@pytest.mark.parametrize("n_requests", [11, 37])
def test_many_requests_decode_together_with_heads_of_128(tmp_path, n_requests):
    """More requests than the mixed cuts hold, heads of 128 (the head size of the tcgen05 prefill attention and of
    the vectorised head norm): prompts of lengths around the 64-key tile and page edges come in two at a time, then
    all requests decode together - a batch that fills its CUDA-graph bucket only in part (rows of padding), with
    and without key splits - and every logit row is compared with the plain implementation."""
    from reinfer_b200.config import Qwen3Config
    from reinfer_b200.engine import Engine
    from reinfer_b200.weights import write_random_model
    raw = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=256, num_attention_heads=4,
               num_key_value_heads=2, head_dim=128, intermediate_size=384, vocab_size=1003, rope_theta=1e6,
               rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=1024)
    d = write_random_model(str(tmp_path / "m"), Qwen3Config.from_dict(raw), seed=9, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(4)
    lens = [1, 2, 63, 64, 65, 127, 128, 129, 200, 31, 300]
    seqs = {f"r{i}": torch.randint(0, 1003, (lens[i % len(lens)] + 6,), generator=g).tolist() for i in range(n_requests)}
    cfg, w = plain.read_model(d)
    want = {r: plain.forward(cfg, w, t, dtype=torch.float32).double() for r, t in seqs.items()}
    names = list(seqs)
    steps = []
    for i in range(0, n_requests, 2):                                   # prompts, two requests a step
        steps.append(([(r, seqs[r][:-6], [len(seqs[r]) - 7]) for r in names[i:i + 2]], []))
    for k in range(6, 0, -1):                                           # then everybody decodes
        steps.append(([(r, [seqs[r][-k]], [0]) for r in names], names if k == 1 else []))
    engine = Engine.from_model_dir(d, dtype="bfloat16", page_size=64, max_tokens=sum(-(-len(t) // 64) * 64 for t in seqs.values()),
                                   max_num_seqs=n_requests)
    got = run_steps(engine, steps)
    assert len(got) == 7 * n_requests
    compare(got, want, TOL["bfloat16"])
    from reinfer_b200 import ops
    assert ops.kernel_error() == 0
