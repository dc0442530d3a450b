"""The tests' own statement of the seeded weight generator, so that the plain implementation
sees the weights of a random model without a file and without the engine's code.

The reference has no random-weights mode; the rule is this engine's.  Its mixing function is
the reference's SplitMix64 (crates/scheduler/src/rng.rs:12-30: GOLDEN_RATIO_64, `mix`,
`splitmix64(x) = mix(x + GOLDEN)`):

    base  = splitmix64(seed XOR fnv1a64(tensor name))
    a, b  = outputs 2i+1 and 2i+2 of the SplitMix64 stream started at base  (i: row-major index)
    value = float32(mean + std * sqrt(-2 ln((a>>11)+1)/2^53) * cos(2 pi (b>>11)/2^53))   in float64

NumPy's unsigned 64-bit arithmetic on the CPU; torch's signed one (wrapping products, masked
shifts) when a CUDA device is given, because a layer of full size has 10^8 elements.  This is
test equipment: nothing of it runs on the engine's path.
"""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch

MASK = (1 << 64) - 1
GOLD = 0x9E3779B97F4A7C15
MUL_A, MUL_B = 0xBF58476D1CE4E5B9, 0x94D049BB133111EB


def mix_int(z: int) -> int:
    z = ((z ^ (z >> 30)) * MUL_A) & MASK
    z = ((z ^ (z >> 27)) * MUL_B) & MASK
    return z ^ (z >> 31)


def name_hash(name: str) -> int:
    """FNV-1a, 64 bits, over the UTF-8 bytes."""
    h = 0xCBF29CE484222325
    for c in name.encode("utf-8"):
        h ^= c
        h = (h * 0x100000001B3) & MASK
    return h


def tensor_base(seed: int, name: str) -> int:
    return mix_int((((seed & MASK) ^ name_hash(name)) + GOLD) & MASK)


def _mix_np(z):
    z = (z ^ (z >> np.uint64(30))) * np.uint64(MUL_A)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(MUL_B)
    return z ^ (z >> np.uint64(31))


def _normal_numpy(n: int, base: int, mean: float, std: float) -> torch.Tensor:
    out = np.empty(n, dtype=np.float32)
    step = 1 << 18
    with np.errstate(over="ignore"):
        for lo in range(0, n, step):
            i = np.arange(lo, min(n, lo + step), dtype=np.uint64)
            a = _mix_np(np.uint64(base) + (np.uint64(2) * i + np.uint64(1)) * np.uint64(GOLD))
            b = _mix_np(np.uint64(base) + (np.uint64(2) * i + np.uint64(2)) * np.uint64(GOLD))
            u1 = ((a >> np.uint64(11)).astype(np.float64) + 1.0) * 2.0 ** -53
            u2 = (b >> np.uint64(11)).astype(np.float64) * 2.0 ** -53
            g = np.sqrt(-2.0 * np.log(u1)) * np.cos(6.283185307179586 * u2)
            out[lo:lo + step] = (mean + std * g).astype(np.float32)
    return torch.from_numpy(out)


def _wrap(v: int) -> int:
    v &= MASK
    return v - (1 << 64) if v >> 63 else v


def _normal_torch(n: int, base: int, mean: float, std: float, device) -> torch.Tensor:
    out = torch.empty(n, dtype=torch.float32, device=device)
    step = 1 << 24

    def mix(z):
        z = (z ^ ((z >> 30) & ((1 << 34) - 1))) * _wrap(MUL_A)
        z = (z ^ ((z >> 27) & ((1 << 37) - 1))) * _wrap(MUL_B)
        return z ^ ((z >> 31) & ((1 << 33) - 1))

    for lo in range(0, n, step):
        i = torch.arange(lo, min(n, lo + step), dtype=torch.int64, device=device)
        two_i_gold = i * _wrap(2 * GOLD)
        a = mix(two_i_gold + _wrap(base + GOLD))
        b = mix(two_i_gold + _wrap(base + 2 * GOLD))
        u1 = (((a >> 11) & ((1 << 53) - 1)).double() + 1.0) * 2.0 ** -53
        u2 = ((b >> 11) & ((1 << 53) - 1)).double() * 2.0 ** -53
        g = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(6.283185307179586 * u2)
        out[lo:lo + step] = (g * std + mean).float()
    return out


def normal(seed: int, name: str, shape, mean: float, std: float, device="cpu") -> torch.Tensor:
    """float32 tensor of `shape`, on `device`."""
    n = int(np.prod(shape)) if len(shape) else 1
    base = tensor_base(seed, name)
    dev = torch.device(device)
    flat = _normal_numpy(n, base, mean, std) if dev.type == "cpu" else _normal_torch(n, base, mean, std, dev)
    return flat.reshape(tuple(shape))


def qwen3_weights(cfg: dict, seed: int, store: str = "float32", device="cpu") -> Dict[str, torch.Tensor]:
    """Every tensor of a random Qwen3 dense model by its checkpoint name (crates/cuda/src/engine.rs:
    3241-3255, 3315-3332): matrices and the embedding N(0, 0.02), norm weights 1 + N(0, 0.05).  With
    store="bfloat16" the float32 values are rounded to bfloat16 (nearest even), as a bfloat16 model
    keeps them.  Returned as float32 tensors on the CPU."""
    h, F, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    QH = cfg["num_attention_heads"]
    KH = cfg.get("num_key_value_heads", QH)
    d = cfg.get("head_dim", h // QH)
    shapes = {"model.embed_tokens.weight": ((V, h), "m"), "model.norm.weight": ((h,), "n")}
    if not cfg.get("tie_word_embeddings"):
        shapes["lm_head.weight"] = ((V, h), "m")
    for i in range(L):
        p = f"model.layers.{i}."
        shapes[p + "input_layernorm.weight"] = ((h,), "n")
        shapes[p + "post_attention_layernorm.weight"] = ((h,), "n")
        shapes[p + "self_attn.q_proj.weight"] = ((QH * d, h), "m")
        shapes[p + "self_attn.k_proj.weight"] = ((KH * d, h), "m")
        shapes[p + "self_attn.v_proj.weight"] = ((KH * d, h), "m")
        shapes[p + "self_attn.o_proj.weight"] = ((h, QH * d), "m")
        shapes[p + "self_attn.q_norm.weight"] = ((d,), "n")
        shapes[p + "self_attn.k_norm.weight"] = ((d,), "n")
        shapes[p + "mlp.gate_proj.weight"] = ((F, h), "m")
        shapes[p + "mlp.up_proj.weight"] = ((F, h), "m")
        shapes[p + "mlp.down_proj.weight"] = ((h, F), "m")
    out = {}
    for name, (shape, how) in shapes.items():
        t = normal(seed, name, shape, 1.0, 0.05, device) if how == "n" else normal(seed, name, shape, 0.0, 0.02, device)
        if store == "bfloat16":
            t = t.to(torch.bfloat16).float()
        out[name] = t.cpu()
    return out
