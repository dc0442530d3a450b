"""Qwen3 dense as a ModelSpec: pre-norm decoder; attention with grouped heads,
per-head q/k RMSNorm (same eps as the layer norms, crates/cuda/src/engine.rs:4124-4147)
and rotary encoding over the whole head (rope_dim = head_dim, crates/arch/src/llama.rs:
380-381); SwiGLU feed-forward; no biases; tied or untied output matrix.  Tensor names
are the checkpoint's (engine.rs:3241-3255, 3315-3332).
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


def build_spec(cfg: Qwen3Config) -> ModelSpec:
    h, eps = cfg.hidden_size, cfg.rms_norm_eps
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            name=f"model.layers.{i}",
            mixer_norm=PartSpec("rmsnorm", {"width": h, "eps": eps}, p + "input_layernorm."),
            mixer=PartSpec("attention", {
                "hidden": h, "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim, "qk_norm": True, "qk_norm_eps": eps,
                "position": {"kind": "rope", "head_dim": cfg.head_dim, "theta": cfg.rope_theta},
                "window": None}, p + "self_attn."),
            ffn_norm=PartSpec("rmsnorm", {"width": h, "eps": eps}, p + "post_attention_layernorm."),
            ffn=PartSpec("swiglu", {"hidden": h, "intermediate": cfg.intermediate_size}, p + "mlp."),
            block="prenorm"))
    tied = cfg.tie_word_embeddings
    return ModelSpec(
        hidden_size=h, vocab_size=cfg.vocab_size,
        embedding=PartSpec("embedding", {"vocab": cfg.vocab_size, "hidden": h}, "model.embed_tokens."),
        layers=tuple(layers),
        final_norm=PartSpec("rmsnorm", {"width": h, "eps": eps}, "model.norm."),
        # untied but absent -> the embedding serves (the reference's GGUF path does the same,
        # crates/cpu/src/model.rs:167-170; its CUDA engine requires lm_head.weight, engine.rs:3254)
        lm_head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": h, "tied": tied,
                                    "fallback": "" if tied else "model.embed_tokens.weight"}, "lm_head."),
        ignorable_tensors=("lm_head.weight",) if tied else ())


def register() -> None:
    register_architecture("Qwen3ForCausalLM", Qwen3Config, build_spec, aliases=("qwen3",))
