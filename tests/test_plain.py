"""The plain implementation checked against itself: its parts against direct formulas,
and properties that any correct forward pass has (no GPU)."""
import math

import torch

import plain_qwen3 as plain
import tiny


def test_rms_norm_formula():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    got = plain.rms_norm(x, w, 0.5)
    r = 1.0 / math.sqrt((9 + 16) / 2 + 0.5)
    assert torch.allclose(got, torch.tensor([[3 * r * 2, 4 * r * 0.5]], dtype=torch.float64))


def test_rope_pairs_and_angles():
    x = torch.arange(8, dtype=torch.float64).reshape(1, 1, 8) + 1
    out = plain.rope_half_split(x, torch.tensor([3]), 100.0)
    for p in range(4):
        ang = 3 * 100.0 ** (-2 * p / 8)
        a, b = x[0, 0, p].item(), x[0, 0, p + 4].item()
        assert abs(out[0, 0, p].item() - (a * math.cos(ang) - b * math.sin(ang))) < 1e-12
        assert abs(out[0, 0, p + 4].item() - (a * math.sin(ang) + b * math.cos(ang))) < 1e-12
    assert torch.equal(plain.rope_half_split(x, torch.tensor([0]), 100.0), x)


def test_attention_is_causal_and_grouped():
    torch.manual_seed(0)
    q, k, v = torch.randn(5, 4, 8).double(), torch.randn(5, 2, 8).double(), torch.randn(5, 2, 8).double()
    full = plain.causal_gqa_attention(q, k, v)
    part = plain.causal_gqa_attention(q[:3], k[:3], v[:3])
    assert torch.allclose(full[:3], part)                        # later tokens do not change earlier ones
    assert torch.allclose(full[0, 1], v[0, 0]) and torch.allclose(full[0, 2], v[0, 1])   # heads 0,1 -> kv 0; 2,3 -> kv 1
    s = (k[:2, 1] @ q[1, 3]) / math.sqrt(8)
    pr = torch.softmax(s, 0)
    assert torch.allclose(full[1, 3], pr[0] * v[0, 1] + pr[1] * v[1, 1])


def test_forward_prefix_property_and_tied_head(tmp_path):
    d = tiny.make_model_dir(str(tmp_path / "a"), "A")
    cfg, w = plain.read_model(d)
    toks = [5, 9, 200, 31, 7, 7, 100]
    full = plain.forward(cfg, w, toks)
    assert full.shape == (7, 256)
    assert torch.allclose(full[:4], plain.forward(cfg, w, toks[:4]), atol=1e-12)
    assert "lm_head.weight" not in w
    g = plain.greedy(cfg, w, toks[:3], 2)
    assert g[0] == int(plain.forward(cfg, w, toks[:3])[-1].argmax())


def test_float32_and_float64_agree(tmp_path):
    d = tiny.make_model_dir(str(tmp_path / "b"), "B")
    cfg, w = plain.read_model(d)
    toks = list(range(20, 45))
    a, b = plain.forward(cfg, w, toks, torch.float64), plain.forward(cfg, w, toks, torch.float32)
    assert (a - b.double()).abs().max().item() < 1e-5 * a.abs().max().item()
