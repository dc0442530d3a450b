"""Safetensors reading/writing and the one error that names everything wrong (no GPU)."""
import json
import os
import struct

import pytest
import torch

import tiny
from reinfer_b200.config import Qwen3Config, resolve_architecture
from reinfer_b200.parts.model import expected_params
from reinfer_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_state, open_model_tensors,
                                  write_random_model, write_safetensors)


def _expected(raw):
    c = Qwen3Config.from_dict(raw)
    return expected_params(resolve_architecture(raw).build_spec(c))


def test_round_trip_all_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
         "d": torch.randn(2, 2).half(), "e": torch.zeros(0, 4)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, metadata={"k": "v"})
    f = SafetensorsFile(p)
    assert sorted(f.names()) == sorted(t) and f.metadata == {"k": "v"}
    for n, v in t.items():
        assert f.dtype(n) == v.dtype and torch.equal(f.tensor(n).clone(), v)


def test_random_model_is_seeded_and_loads(tmp_path):
    d1 = write_random_model(str(tmp_path / "m1"), Qwen3Config.from_dict(tiny.TINY_B), 1, torch.float32)
    d2 = write_random_model(str(tmp_path / "m2"), Qwen3Config.from_dict(tiny.TINY_B), 1, torch.float32)
    d3 = write_random_model(str(tmp_path / "m3"), Qwen3Config.from_dict(tiny.TINY_B), 2, torch.float32)
    exp = _expected(tiny.TINY_B)
    s1, s2, s3 = (load_state(d, exp, torch.float32, "cpu") for d in (d1, d2, d3))
    assert all(torch.equal(s1[k], s2[k]) for k in s1)
    assert not torch.equal(s1["model.embed_tokens.weight"], s3["model.embed_tokens.weight"])
    w = s1["model.layers.0.self_attn.q_proj.weight"]
    assert abs(w.std().item() - 0.02) < 0.002
    n = s1["model.norm.weight"]
    assert abs(n.mean().item() - 1.0) < 0.03
    assert json.load(open(os.path.join(d1, "config.json")))["num_attention_heads"] == 6


def test_storage_rule(tmp_path):
    """16-bit tensors are kept as bfloat16, 32-bit ones stay 32-bit; float32 mode widens everything."""
    d = write_random_model(str(tmp_path / "m"), Qwen3Config.from_dict(tiny.TINY_A), 0, torch.bfloat16)
    f, _ = open_model_tensors(d)["model.norm.weight"]
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()
    tensors["model.layers.0.mlp.up_proj.weight"] = tensors["model.layers.0.mlp.up_proj.weight"].half()
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    exp = _expected(tiny.TINY_A)
    s = load_state(d, exp, torch.bfloat16, "cpu")
    assert s["model.norm.weight"].dtype == torch.float32
    assert s["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    assert s["model.embed_tokens.weight"].dtype == torch.bfloat16
    s32 = load_state(d, exp, torch.float32, "cpu")
    assert all(v.dtype == torch.float32 for v in s32.values())


def test_one_error_lists_everything(tmp_path):
    d = write_random_model(str(tmp_path / "m"), Qwen3Config.from_dict(tiny.TINY_B), 1, torch.float32)
    f, _ = open_model_tensors(d)["model.norm.weight"]
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.layers.2.self_attn.k_norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(96, 192)
    tensors["model.norm.weight"] = torch.zeros(96, dtype=torch.int32)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        load_state(d, _expected(tiny.TINY_B), torch.float32, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.layers.2.self_attn.k_norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (192, 96), (96, 192))]
    assert err.wrong_dtype[0][0] == "model.norm.weight"
    for word in ("missing", "unexpected", "wrong shape", "expected [192, 96] got [96, 192]"):
        assert word in str(err)


def test_tied_and_absent_output_matrix(tmp_path):
    d = write_random_model(str(tmp_path / "a"), Qwen3Config.from_dict(tiny.TINY_A), 0, torch.float32)
    assert "lm_head.weight" not in open_model_tensors(d)
    # a tied checkpoint that still carries lm_head.weight is accepted
    f, _ = open_model_tensors(d)["model.norm.weight"]
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    spec = resolve_architecture(tiny.TINY_A).build_spec(Qwen3Config.from_dict(tiny.TINY_A))
    load_state(d, expected_params(spec), torch.float32, "cpu", ignorable=spec.ignorable_tensors)
    # untied but absent: optional, the embedding will serve
    d2 = write_random_model(str(tmp_path / "b"), Qwen3Config.from_dict(tiny.TINY_B), 1, torch.float32)
    f, _ = open_model_tensors(d2)["model.norm.weight"]
    tensors = {n: f.tensor(n).clone() for n in f.names() if n != "lm_head.weight"}
    write_safetensors(os.path.join(d2, "model.safetensors"), tensors)
    s = load_state(d2, _expected(tiny.TINY_B), torch.float32, "cpu")
    assert "lm_head.weight" not in s


def test_sharded_folder(tmp_path):
    d = write_random_model(str(tmp_path / "m"), Qwen3Config.from_dict(tiny.TINY_A), 0, torch.float32)
    f, _ = open_model_tensors(d)["model.norm.weight"]
    names = sorted(f.names())
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    wm = {}
    for shard, ns in shards.items():
        write_safetensors(os.path.join(d, shard), {n: f.tensor(n).clone() for n in ns})
        wm.update({n: shard for n in ns})
    ref = load_state(d, _expected(tiny.TINY_A), torch.float32, "cpu")
    os.remove(os.path.join(d, "model.safetensors"))
    json.dump({"weight_map": wm}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    got = load_state(d, _expected(tiny.TINY_A), torch.float32, "cpu")
    assert all(torch.equal(ref[k], got[k]) for k in ref)


def test_broken_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 2) + b"{x")
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="needs 16"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="outside"):
        SafetensorsFile(str(p))
    with pytest.raises(FileNotFoundError):
        open_model_tensors(str(tmp_path / "nothing"))


def ulps_apart(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance of float32 values in units in the last place (bit patterns as ordered integers)."""
    def key(t):
        i = t.contiguous().view(torch.int32).long()
        return torch.where(i < 0, -(i & 0x7FFFFFFF), i)
    return (key(a) - key(b)).abs()


def same_up_to_library_rounding(a: torch.Tensor, b: torch.Tensor) -> None:
    """Two evaluations of the generator's formula: equal, but for the rare element whose float64
    logarithm or cosine differs in its last bit between two mathematical libraries and lies on a
    float32 rounding boundary (one unit in the last place, a few elements in 10^8)."""
    apart = ulps_apart(a.float(), b.float())
    assert int(apart.max()) <= 1
    assert int((apart > 0).sum()) <= max(1, a.numel() // 1_000_000)


@pytest.mark.parametrize("which", ["A", "B"])
def test_random_weights_are_the_stated_function_of_seed_name_and_index(tmp_path, which):
    """The package's generator, the folder it writes and the tests' own statement of the rule give the
    same tensors; a tensor does not depend on the others, nor on the pieces it is drawn in."""
    import plain_random
    from reinfer_b200.weights import random as rnd
    from reinfer_b200.weights import random_state
    raw, seed, _ = tiny.TINY[which]
    exp = _expected(raw)
    drawn = random_state(exp, seed, torch.float32, "cpu")
    want = plain_random.qwen3_weights(raw, seed)
    assert sorted(drawn) == sorted(want)
    for name in want:
        assert drawn[name].shape == want[name].shape
        same_up_to_library_rounding(drawn[name], want[name])
    d = write_random_model(str(tmp_path / "m"), Qwen3Config.from_dict(raw), seed, torch.float32)
    stored = load_state(d, exp, torch.float32, "cpu")
    assert all(torch.equal(stored[k], drawn[k]) for k in drawn)
    # bfloat16: the same float32 values, rounded once
    b16 = random_state(exp, seed, torch.bfloat16, "cpu")
    want16 = plain_random.qwen3_weights(raw, seed, store="bfloat16")
    for name in want16:
        assert int((b16[name].float() != want16[name]).sum()) <= 1
    # one tensor alone, and a piece of it from the middle
    name = "model.layers.1.mlp.down_proj.weight"
    alone = random_state({name: exp[name]}, seed, torch.float32, "cpu")[name]
    assert torch.equal(alone, drawn[name])
    base = rnd.stream_base(seed, name)
    assert base == plain_random.tensor_base(seed, name)
    whole = rnd.normal_cpu((alone.numel(),), base, 0.0, 0.02)
    assert torch.equal(whole.reshape(alone.shape), alone)
    assert rnd.stream_base(seed + 1, name) != base and rnd.stream_base(seed, name + "x") != base


def test_random_weights_have_the_stated_moments():
    from reinfer_b200.weights import random as rnd
    t = rnd.normal_cpu((1 << 20,), rnd.stream_base(3, "t"), 0.0, 0.02).double()
    assert abs(t.mean().item()) < 1e-4 and abs(t.std().item() - 0.02) < 1e-4
    assert abs(((t / 0.02) ** 4).mean().item() - 3.0) < 0.05            # a normal's fourth moment
    n = rnd.normal_cpu((1 << 16,), rnd.stream_base(3, "n"), 1.0, 0.05).double()
    assert abs(n.mean().item() - 1.0) < 1e-3 and abs(n.std().item() - 0.05) < 1e-3
    i = rnd.ints_cpu((1 << 16,), rnd.stream_base(3, "i"))
    assert i.dtype == torch.int32 and int(i.min()) >= 0 and int(i.max()) < (1 << 15) and int(i.max()) > 32000
