"""The engine at the layer sizes of the three full-size configurations (Qwen3-4B, 8B and 32B: every
hidden size, head count, group width and feed-forward width of them; two layers each, and a small odd
vocabulary, because the plain implementation runs them on the CPU), with weights that come from the
seeded generator on both sides and never pass through a file: the engine draws them on the device, the
plain implementation from the tests' own statement of the rule."""
from __future__ import annotations

import pytest
import torch

import plain_qwen3 as plain
import plain_random
import tiny
from test_engine_gpu import TOL, compare, run_steps
from test_weights import same_up_to_library_rounding

pytestmark = pytest.mark.gpu

VOCAB = 8009
COMMON = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, head_dim=128, vocab_size=VOCAB,
              rope_theta=1e6, rms_norm_eps=1e-6, max_position_embeddings=8192)
SHAPES = {
    "4b": dict(COMMON, hidden_size=2560, num_attention_heads=32, num_key_value_heads=8, intermediate_size=9728,
               tie_word_embeddings=True),
    "8b": dict(COMMON, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, intermediate_size=12288,
               tie_word_embeddings=False),
    "32b": dict(COMMON, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, intermediate_size=25600,
                tie_word_embeddings=False),
}
SEED = 3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_device_generator_is_the_stated_function(dtype):
    """The kernel that draws a model's weights against the tests' own statement of the rule (evaluated by
    torch on the device and by NumPy on the CPU): whole tensors, odd sizes, both kinds of initialisation."""
    from reinfer_b200.weights import random as rnd
    for name, shape, mean, std in (("model.layers.1.mlp.down_proj.weight", (1031, 517), 0.0, 0.02),
                                   ("model.norm.weight", (4099,), 1.0, 0.05),
                                   ("model.embed_tokens.weight", (3, 5), 0.0, 0.02),
                                   ("lm_head.weight", (2048, 4096), 0.0, 0.02)):
        got = rnd.normal(shape, SEED, name, mean, std, dtype, "cuda")
        assert got.dtype == dtype and tuple(got.shape) == shape
        want_dev = plain_random.normal(SEED, name, shape, mean, std, device="cuda")
        want_cpu = plain_random.normal(SEED, name, shape, mean, std, device="cpu")
        same_up_to_library_rounding(want_dev.cpu(), want_cpu)
        if dtype == torch.float32:
            same_up_to_library_rounding(got.cpu(), want_cpu)
        else:
            # rounded once more, to bfloat16: an element moves only if its float32 value did
            assert int((got.float().cpu() != want_cpu.to(torch.bfloat16).float()).sum()) <= 1
    ints = rnd.ints((1000,), SEED, "table", "cuda")
    assert torch.equal(ints.cpu(), rnd.ints_cpu((1000,), rnd.stream_base(SEED, "table")))


_truths = {}


def shape_truth(shape: str, store: str, seqs):
    """The plain implementation's logits (float32 arithmetic on the CPU) for the model of this shape and seed."""
    key = (shape, store, tuple((r, tuple(t)) for r, t in seqs.items()))
    if key not in _truths:
        cfg = SHAPES[shape]
        w = plain_random.qwen3_weights(cfg, SEED, store=store, device="cuda")
        _truths[key] = {r: plain.forward(cfg, w, t, dtype=torch.float32).double() for r, t in seqs.items()}
    return _truths[key]


def shape_engine(shape: str, dtype: str, pool_tokens: int, max_num_seqs: int = 4, **kw):
    from reinfer_b200.config import Qwen3Config
    from reinfer_b200.engine import Engine
    return Engine.from_config(Qwen3Config.from_dict(SHAPES[shape]), seed=SEED, dtype=dtype, page_size=16,
                              max_tokens=pool_tokens, max_num_seqs=max_num_seqs, **kw)


def random_sequences(lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"s{i}": torch.randint(0, VOCAB, (n,), generator=g).tolist() for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", list(SHAPES))
def test_full_size_layer_shapes(shape, dtype):
    """Whole prompts and the mixed cut (up to four live requests, a pool of exactly the pages the steps need,
    so that later requests get the pages of finished ones) against the plain implementation."""
    seqs = random_sequences([150, 70, 300, 33, 129], seed=1)
    want = shape_truth(shape, dtype, seqs)
    for cut in (tiny.cut_whole, tiny.cut_mixed):
        steps = cut(seqs)
        engine = shape_engine(shape, dtype, tiny.pool_tokens_needed(steps, 16))
        owners = tiny.PageOwners(engine.cache)
        got = run_steps(engine, steps, owners)
        assert len(got) == sum(len(t) for t in seqs.values())
        compare(got, want, TOL[dtype])
        if cut is tiny.cut_mixed:
            assert len(owners.reused) >= 4
        engine.check_status()
        del engine
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_large_portions_beside_decoding_requests(dtype):
    """Steps as a serving run at full layer sizes composes them: two prompts in portions of 300 to 700 tokens
    that continue from cached pages (and one of two tokens), beside eight requests that decode one token each;
    every row of every step against the plain implementation.  The pool holds exactly what the steps need, and
    a request that came and went before has left its pages behind in another order."""
    shape = "8b"
    gone = random_sequences([200], seed=5)["s0"]
    big = random_sequences([1053, 1044], seed=6)
    small = random_sequences([20 + 11 * i + 4 for i in range(8)], seed=7)
    seqs = {"p0": big["s0"], "p1": big["s1"], **{f"d{i}": small[f"s{i}"] for i in range(8)}}
    want = shape_truth(shape, dtype, seqs)
    every = lambda tokens: list(range(len(tokens)))
    decode = lambda k, end=False: [(r, [seqs[r][len(seqs[r]) - 4 + k]], [0]) for r in seqs if r.startswith("d")]
    p0, p1 = seqs["p0"], seqs["p1"]
    steps = [
        ([(r, seqs[r][:-4], every(seqs[r][:-4])) for r in seqs if r.startswith("d")], []),
        ([("p0", p0[:350], every(p0[:350])), ("p1", p1[:410], every(p1[:410]))] + decode(0), []),
        ([("p0", p0[350:1050], every(p0[350:1050])), ("p1", p1[410:710], every(p1[410:710]))] + decode(1), []),
        ([("p0", p0[1050:1052], [0, 1]), ("p1", p1[710:1043], every(p1[710:1043]))] + decode(2), []),
        ([("p0", p0[1052:], [0]), ("p1", p1[1043:], [0])] + decode(3), list(seqs)),
    ]
    pool = max(tiny.pool_tokens_needed(steps, 16), -(-len(gone) // 16) * 16)
    engine = shape_engine(shape, dtype, pool, max_num_seqs=10)
    from reinfer_b200.engine import StepEntry
    for lo in range(0, 100, 20):                       # two requests that grow in turns: their pages interleave
        engine.step([StepEntry("gone", gone[lo:lo + 20], []), StepEntry("gone2", gone[100 + lo:120 + lo], [])])
    engine.finish("gone")
    engine.finish("gone2")
    owners = tiny.PageOwners(engine.cache)
    got = run_steps(engine, steps, owners)
    assert len(got) == sum(len(t) for t in seqs.values())
    compare(got, want, TOL[dtype])
    assert engine.cache.free_pages() == engine.cache.total_pages()
    engine.check_status()
