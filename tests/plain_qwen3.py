"""A plain, slow restatement of the Qwen3 dense forward pass: whole sequences, no
cache, one function per part, torch on the CPU only.  It shares no code with
`reinfer_b200`; tests compare the engine with it.

The reference's model code is Rust plus CUDA; the Rust cannot be compiled here, so
the forward pass as a whole rests on the reference's formulas: every function cites
the file and line whose arithmetic it restates.  The parts, however, are held
against the reference's own CUDA kernels: tests/golden/make_golden.py compiles those
kernels unchanged and records what they compute (RMSNorm, the rotation, per-head
norm before rotation, SwiGLU, the masked softmax, grouped decode attention over a
paged cache, the sampler's draws), and tests/test_golden.py compares the functions
below with those records.  `dtype` is the precision it computes in: float64 by
default, so that it is a truth for the 32-bit engine too.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np
import torch


# ---------------------------------------------------------------- file reading
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """Tensors of one safetensors file as float64 (integers as int64).
    Format: crates/safetensors/src/lib.rs:62-124 (u64 LE header length, JSON
    header with dtype/shape/data_offsets, raw little-endian data)."""
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, en = e["data_offsets"]
        buf = data[b:en]
        dt = e["dtype"]
        if dt == "F32":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<f4").copy()).double()
        elif dt == "F16":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<f2").copy()).double()
        elif dt == "BF16":
            u = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).copy()).double()
        elif dt in ("I32", "I64"):
            t = torch.from_numpy(np.frombuffer(buf, dtype="<i4" if dt == "I32" else "<i8").copy()).long()
        else:
            raise ValueError(f"{name}: dtype {dt}")
        out[name] = t.reshape(e["shape"])
    return out


def read_model(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ------------------------------------------------------------------- the parts
def embed(table: torch.Tensor, tokens: List[int]) -> torch.Tensor:
    """x[t,:] = E[token[t],:]  (crates/cuda/kernels/dense_kernels.cu:329-336)."""
    return torch.stack([table[t] for t in tokens])


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w over the last axis; eps inside the root; plain
    weight (crates/kernels/src/refs.rs:10-18, dense_kernels.cu:59-88)."""
    ms = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x / torch.sqrt(ms + eps) * w


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = x W^T with W stored [out, in], no bias (crates/cuda/src/engine.rs:4090-4119)."""
    return x @ w.t()


def rope_half_split(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotation of the pairs (p, p+d/2): angle = pos * theta^(-2p/d)
    (refs.rs:25-37; dense_kernels.cu:127-170).  x: [S, heads, d]."""
    d = x.shape[-1]
    half = d // 2
    p = torch.arange(half, dtype=x.dtype)
    inv = torch.tensor(theta, dtype=x.dtype) ** (-(2.0 * p) / d)
    ang = positions.to(x.dtype)[:, None] * inv[None, :]          # [S, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def head_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over each head row of length d with one weight [d] for all heads, after
    the projection and before the rotation, same eps as the layer norms
    (dense_kernels.cu:92-123; engine.rs:4124-4147)."""
    return rms_norm(x, w, eps)


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """q [S,QH,d], k/v [S,KH,d]; query head hq reads kv head hq // (QH/KH); scores
    q.k/sqrt(d) over keys t <= own position, softmax with max subtracted, weighted sum
    of v (crates/cuda/tests/engine_vs_cpu.rs:208-237; decode_flash_kernels.cu:212-349)."""
    S, QH, d = q.shape
    KH = k.shape[1]
    group = QH // KH
    out = torch.zeros_like(q)
    scale = 1.0 / math.sqrt(d)
    for h in range(QH):
        kh = h // group
        for s in range(S):
            sc = (k[: s + 1, kh] @ q[s, h]) * scale
            pr = torch.exp(sc - sc.max())
            out[s, h] = (pr[:, None] * v[: s + 1, kh]).sum(0) / pr.sum()
    return out


def swiglu_ffn(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """down( g/(1+exp(-g)) * u ), g = x Wg^T, u = x Wu^T (engine.rs:4288-4314;
    dense_kernels.cu:236-248)."""
    g, u = linear(x, wg), linear(x, wu)
    return linear(g / (1.0 + torch.exp(-g)) * u, wd)


def attention_block(x, w, prefix, cfg, positions):
    """Projections, per-head norm, rotation, attention, output projection
    (engine.rs:4090-4269, the order of its launches)."""
    QH, KH = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"])
    d = cfg.get("head_dim", cfg["hidden_size"] // QH)
    eps, theta = cfg.get("rms_norm_eps", 1e-5), cfg.get("rope_theta", 1e6)
    S = x.shape[0]
    q = linear(x, w[prefix + "q_proj.weight"]).reshape(S, QH, d)
    k = linear(x, w[prefix + "k_proj.weight"]).reshape(S, KH, d)
    v = linear(x, w[prefix + "v_proj.weight"]).reshape(S, KH, d)
    q = head_norm(q, w[prefix + "q_norm.weight"], eps)
    k = head_norm(k, w[prefix + "k_norm.weight"], eps)
    q = rope_half_split(q, positions, theta)
    k = rope_half_split(k, positions, theta)
    a = causal_gqa_attention(q, k, v).reshape(S, QH * d)
    return linear(a, w[prefix + "o_proj.weight"])


def decoder_layer(x, w, i, cfg, positions):
    """x += attn(norm(x)); x += ffn(norm(x))  (engine.rs:4071-4333)."""
    p = f"model.layers.{i}."
    eps = cfg.get("rms_norm_eps", 1e-5)
    x = x + attention_block(rms_norm(x, w[p + "input_layernorm.weight"], eps), w, p + "self_attn.", cfg, positions)
    x = x + swiglu_ffn(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps),
                       w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return x


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int],
            dtype=torch.float64) -> torch.Tensor:
    """Logits [S, vocab] of the whole sequence (engine.rs:4337-4347 for the end: final
    norm, then the output matrix; the embedding serves as output matrix when
    `tie_word_embeddings` is set or `lm_head.weight` is absent)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    positions = torch.arange(len(tokens))
    x = embed(w["model.embed_tokens.weight"], tokens)
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, i, cfg, positions)
    x = rms_norm(x, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-5))
    head = w["model.embed_tokens.weight"] if (cfg.get("tie_word_embeddings") or "lm_head.weight" not in w) \
        else w["lm_head.weight"]
    return linear(x, head)


def greedy(cfg, weights, prompt: List[int], n: int, dtype=torch.float64) -> List[int]:
    """n greedy tokens, first maximum on ties (bench/referee/llama_referee.cpp:8-10)."""
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(forward(cfg, weights, toks, dtype)[-1]).item()))
    return toks[len(prompt):]
