"""The plain implementation against numbers that the reference's own kernels produced.

tests/golden/reference_kernels.json was written by tests/golden/make_golden.py, which compiles
crates/cuda/kernels/{diff,dense,decode_gqa,sampler}_kernel(s).cu of LeonRust/reinfer unchanged and runs
them on a GPU.  Every tolerance below is the rounding of the reference's own storage (float32 or float16
results compared with float64 arithmetic), not slack for a different formula: a moved eps, a `1 + w`
weight, another pairing of the rotation, norm after rotation instead of before, or another constant in
the random stream would miss these by orders of magnitude.
"""
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_kernels.json")


@pytest.fixture(scope="module")
def golden():
    with open(PATH) as f:
        return json.load(f)["cases"]


def f64(v):
    return torch.tensor([float(x) for x in v], dtype=torch.float64)


def from_f16_bits(bits):
    return torch.from_numpy(np.asarray(bits, dtype=np.uint16).view(np.float16).astype(np.float64))


def test_rms_norm_matches_the_reference_kernel(golden):
    for c in golden["rms_norm_row"]:
        got = plain.rms_norm(f64(c["x"]), f64(c["w"]), c["eps"])
        want = f64(c["out"])
        assert (got - want).abs().max().item() <= 2e-6 * want.abs().max().item()
        # the alternatives a wrong reading would give are far away
        x, w = f64(c["x"]), f64(c["w"])
        outside = x / (torch.sqrt((x * x).mean()) + c["eps"]) * w
        plus_one = x / torch.sqrt((x * x).mean() + c["eps"]) * (1 + w)
        assert (plus_one - want).abs().max().item() > 1e-2


def test_rotation_matches_the_reference_kernel(golden):
    for c in golden["rope_row"]:
        half = c["half"]
        x = f64(c["x"]).reshape(1, 1, 2 * half)
        got = plain.rope_half_split(x, torch.tensor([c["pos"]]), c["eta"]).reshape(-1)
        want = f64(c["out"])
        # the kernel forms pos * powf(eta, ..) and its sine and cosine in float32: the angle is off by up to
        # ~1e-7 * pos radians, the result by that times |x|
        tol = 4e-6 + 3e-7 * c["pos"]
        assert (got - want).abs().max().item() <= tol * max(1.0, want.abs().max().item()), c["pos"]
        if c["pos"] > 0:
            x1 = x.reshape(-1)
            interleaved = torch.stack([x1[0::2], x1[1::2]])             # pairs (2p, 2p+1) instead of (p, p + half)
            assert not torch.allclose(interleaved.reshape(-1), want, atol=1e-3)


def test_masked_softmax_matches_the_reference_kernel(golden):
    c = golden["masked_softmax_row"][0]
    x = torch.tensor([float("-inf") if v == "-inf" else float(v) for v in c["x"]], dtype=torch.float64)
    e = torch.exp(x - x.max())                                            # what plain.causal_gqa_attention does with its scores
    got = e / e.sum()
    want = f64(c["out"])
    assert (got - want).abs().max().item() <= 2e-7
    assert all(want[i] == 0 for i in (3, 17, 49))


def test_head_norm_comes_before_rotation_as_in_the_reference(golden):
    c = golden["head_norm_then_rope_f16"][0]
    rows, n = c["rows"], c["n"]
    x = from_f16_bits(c["x_bits"]).reshape(rows, n)
    w = from_f16_bits(c["w_bits"])
    normed = plain.head_norm(x, w, c["eps"])
    want_normed = from_f16_bits(c["normed_bits"]).reshape(rows, n)
    assert (normed - want_normed).abs().max().item() <= 1.5e-3 * want_normed.abs().max().item()    # float16 storage
    got = plain.rope_half_split(normed.reshape(1, rows, n), torch.tensor([c["pos"]]), c["eta"]).reshape(rows, n)
    want = from_f16_bits(c["out_bits"]).reshape(rows, n)
    assert (got - want).abs().max().item() <= 3e-3 * want.abs().max().item()
    # rotation first and norm second gives the same (a rotation keeps a row's norm) only with a weight of ones;
    # with the real weight it is another result
    other = plain.head_norm(plain.rope_half_split(x.reshape(1, rows, n), torch.tensor([c["pos"]]), c["eta"]).reshape(rows, n), w, c["eps"])
    assert (other - want).abs().max().item() > 1e-2


def test_swiglu_matches_the_reference_kernels(golden):
    c = golden["swiglu"][0]
    g, u = f64(c["gate"]), f64(c["up"])
    got = g / (1.0 + torch.exp(-g)) * u                                   # the activation of plain.swiglu_ffn
    assert (got - f64(c["out"])).abs().max().item() <= 2e-6 * f64(c["out"]).abs().max().item()
    ident = torch.eye(len(g), dtype=torch.float64)
    through_ffn = plain.swiglu_ffn(torch.ones(1, 1, dtype=torch.float64), g.reshape(-1, 1), u.reshape(-1, 1), ident)
    assert (through_ffn.reshape(-1) - f64(c["out"])).abs().max().item() <= 2e-6 * f64(c["out"]).abs().max().item()
    g16, u16 = from_f16_bits(c["gate_bits"]), from_f16_bits(c["up_bits"])
    want16 = from_f16_bits(c["out_bits"])
    assert ((g16 / (1.0 + torch.exp(-g16)) * u16) - want16).abs().max().item() <= 1e-3 * want16.abs().max().item()


def test_grouped_attention_matches_the_reference_decode_kernel(golden):
    c = golden["decode_step_gqa"][0]
    QH, KH, d, n = c["QH"], c["KH"], c["d"], c["kv_len"]
    q_scaled = from_f16_bits(c["q_scaled_bits"]).reshape(QH, d)
    k = from_f16_bits(c["k_bits"]).reshape(n, KH, d)
    v = from_f16_bits(c["v_bits"]).reshape(n, KH, d)
    # the plain function scales by 1/sqrt(d) itself and computes every position; the kernel got q already scaled and
    # computes the last one: hand the plain function q * sqrt(d) at the last position
    q = torch.zeros(n, QH, d, dtype=torch.float64)
    q[-1] = q_scaled * math.sqrt(d)
    got = plain.causal_gqa_attention(q, k, v)[-1]
    want = from_f16_bits(c["out_bits"]).reshape(QH, d)
    assert (got - want).abs().max().item() <= 1.5e-3 * want.abs().max().item()
    # query head h reads kv head h // (QH / KH): with the heads interleaved instead the result is another
    wrong = plain.causal_gqa_attention(q[:, [0, 2, 4, 1, 3, 5]], k, v)[-1]
    assert (wrong - want).abs().max().item() > 1e-2
