"""Configuration parsing and the architecture registry (no GPU)."""
import json

import pytest

import tiny
from reinfer_b200.config import (InvalidValue, MissingKey, Qwen3Config, UnknownArchitecture,
                                 load_config, register_architecture, resolve_architecture, resolve_eos,
                                 unregister_architecture)


def test_parses_own_keys_and_defaults():
    c = Qwen3Config.from_dict(tiny.TINY_B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (3, 96, 6, 2, 32)
    assert c.vocab_size == 311 and c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and not c.tie_word_embeddings
    d = dict(tiny.TINY_A)
    for k in ("num_key_value_heads", "head_dim", "rope_theta", "rms_norm_eps", "tie_word_embeddings"):
        d.pop(k)
    c = Qwen3Config.from_dict(d)
    assert c.num_key_value_heads == 4 and c.head_dim == 16          # kv heads = q heads, head_dim = hidden / heads
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and c.tie_word_embeddings is False


def test_round_trip():
    c = Qwen3Config.from_dict(tiny.TINY_B)
    assert Qwen3Config.from_dict(c.to_dict()) == c


@pytest.mark.parametrize("key", ["max_position_embeddings", "num_hidden_layers", "hidden_size", "intermediate_size",
                                 "vocab_size", "num_attention_heads"])
def test_missing_key(key):
    d = dict(tiny.TINY_A)
    d.pop(key)
    with pytest.raises(MissingKey) as e:
        Qwen3Config.from_dict(d)
    assert key in str(e.value)


@pytest.mark.parametrize("patch,key", [
    ({"num_attention_heads": 0}, "num_attention_heads"),
    ({"num_key_value_heads": 0}, "num_key_value_heads"),
    ({"num_key_value_heads": 8}, "num_key_value_heads"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),          # 4 query heads over 3 kv heads
    ({"head_dim": 15}, "head_dim"),
    ({"rope_theta": 0}, "rope_theta"),
    ({"rope_theta": float("inf")}, "rope_theta"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"use_sliding_window": True}, "use_sliding_window"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"vocab_size": -3}, "vocab_size"),
])
def test_invalid_values(patch, key):
    d = dict(tiny.TINY_A)
    d.update(patch)
    with pytest.raises(InvalidValue) as e:
        Qwen3Config.from_dict(d)
    assert e.value.key == key


def test_underivable_head_dim():
    d = dict(tiny.TINY_A, hidden_size=66)
    d.pop("head_dim")
    with pytest.raises(InvalidValue):
        Qwen3Config.from_dict(d)


def test_registry_by_architectures_then_model_type(tmp_path):
    assert resolve_architecture({"architectures": ["Qwen3ForCausalLM"]}).name == "Qwen3ForCausalLM"
    assert resolve_architecture({"model_type": "qwen3"}).name == "Qwen3ForCausalLM"
    with pytest.raises(UnknownArchitecture) as e:
        resolve_architecture({"architectures": ["LlamaForCausalLM"]})
    assert "Qwen3ForCausalLM" in str(e.value)
    with pytest.raises(MissingKey):
        resolve_architecture({})
    (tmp_path / "config.json").write_text(json.dumps(tiny.TINY_A))
    arch, cfg = load_config(str(tmp_path))
    assert arch.name == "Qwen3ForCausalLM" and cfg.hidden_size == 64


def test_registering_another_architecture():
    class Cfg:
        @classmethod
        def from_dict(cls, d):
            return cls()
    register_architecture("ToyArch", Cfg, lambda c: None, aliases=("toy",))
    try:
        assert resolve_architecture({"model_type": "toy"}).config_cls is Cfg
    finally:
        unregister_architecture("ToyArch")
    with pytest.raises(UnknownArchitecture):
        resolve_architecture({"model_type": "toy"})


def test_eos_resolution(tmp_path):
    c = Qwen3Config.from_dict(dict(tiny.TINY_A, eos_token_id=[7, 9]))
    assert resolve_eos(c) == (7, 9)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [11, 12]}))
    assert resolve_eos(c, str(tmp_path)) == (11, 12)
    assert resolve_eos(Qwen3Config.from_dict(tiny.TINY_A)) == (151645,)


def test_spec_is_data_with_every_size_from_config():
    from reinfer_b200.parts.model import expected_params
    for raw in (tiny.TINY_A, tiny.TINY_B):
        c = Qwen3Config.from_dict(raw)
        spec = resolve_architecture(raw).build_spec(c)
        assert len(spec.layers) == c.num_hidden_layers
        m = spec.layers[0].mixer.params
        assert (m["q_heads"], m["kv_heads"], m["head_dim"]) == (c.num_attention_heads, c.num_key_value_heads, c.head_dim)
        assert m["position"]["theta"] == c.rope_theta and m["qk_norm_eps"] == c.rms_norm_eps
        e = expected_params(spec)
        assert e["model.layers.0.self_attn.q_proj.weight"].shape == (c.num_attention_heads * c.head_dim, c.hidden_size)
        assert e["model.layers.0.mlp.down_proj.weight"].shape == (c.hidden_size, c.intermediate_size)
        assert ("lm_head.weight" in e) == (not c.tie_word_embeddings)
