"""Causal attention with grouped heads over the paged cache
(crates/cuda/src/engine.rs:4090-4281 in launch order): fused q/k/v projection, optional
per-head RMSNorm of q and k with one weight [d] for all heads (dense_kernels.cu:92-123),
position encoding, append of k and v to the request's pages, softmax(q k^T / sqrt(d)) v
over the keys up to the token's own position (optionally only the last `window`), output
projection added into the residual stream.  All sizes and constants are parameters.

The q, k and v matrices are concatenated by rows once at load into `[(QH+2KH) d, h]`
(one product for three; the reference keeps a fused copy AND the separate ones,
engine.rs:3268-3319).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..weights.params import ParamSpec
from .base import Mixer, PagedKVSpec, RowScaled, build_part, register_part
from .linear import matmul, matmul_into_residual, takes_row_scaled
from .spec import PartSpec


class Attention(Mixer):
    def __init__(self, hidden: int, q_heads: int, kv_heads: int, head_dim: int,
                 qk_norm: bool = False, qk_norm_eps: float = 1e-6, position: Optional[dict] = None,
                 window: Optional[int] = None, scale: Optional[float] = None):
        self.hidden, self.QH, self.KH, self.d = int(hidden), int(q_heads), int(kv_heads), int(head_dim)
        if self.QH <= 0 or self.KH <= 0 or self.QH % self.KH:
            raise ValueError(f"attention: {self.QH} query heads over {self.KH} kv heads")
        self.qk_norm, self.eps = bool(qk_norm), float(qk_norm_eps)
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.d)   # engine.rs:4150-4160
        pos = dict(position) if position else {"kind": "none"}
        kind = pos.pop("kind")
        self.position = build_part("position", PartSpec(kind, pos))
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None

    # ---- declarations ------------------------------------------------------
    def param_specs(self):
        h, d = self.hidden, self.d
        out = {"q_proj.weight": ParamSpec((self.QH * d, h)),
               "k_proj.weight": ParamSpec((self.KH * d, h)),
               "v_proj.weight": ParamSpec((self.KH * d, h)),
               "o_proj.weight": ParamSpec((h, self.QH * d))}
        if self.qk_norm:
            out["q_norm.weight"] = ParamSpec((d,), init="norm")
            out["k_norm.weight"] = ParamSpec((d,), init="norm")
        return out

    def cache_spec(self):
        return PagedKVSpec(self.KH, self.d, self.window)

    def bind(self, tensors):
        q, k, v = tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]
        if not (q.dtype == k.dtype == v.dtype):
            q, k, v = q.float(), k.float(), v.float()
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"]
        if self.qk_norm:
            self.q_norm_w, self.k_norm_w = tensors["q_norm.weight"], tensors["k_norm.weight"]
            if self.q_norm_w.dtype != self.k_norm_w.dtype:
                self.q_norm_w, self.k_norm_w = self.q_norm_w.float(), self.k_norm_w.float()

    def prepare(self, device, dtype) -> None:
        if self.position is not None:
            self.position.prepare(device)

    @property
    def takes_row_scaled(self) -> bool:
        """The first product (q, k, v) can apply the factor of rows that the norm left without it."""
        return takes_row_scaled(self.w_qkv)

    def decode_plan(self, live: int, largest_tiles: int, total_tiles: int):
        """What a decode step of `live` requests, whose keys fill `total_tiles` 64-key tiles (the longest
        `largest_tiles`), fixes beyond its shapes: in how many parts the attention splits a request's keys.  A captured
        step is made for one plan and reused by every batch that asks for the same (the engine keys its graphs by it)."""
        pairs = self.KH * ((self.QH // self.KH) // ops.fa_group_chunk(self.QH // self.KH))
        return ops.decode_splits(max(1, live) * pairs, max(1, largest_tiles), head_dim=self.d, total_tiles=max(1, total_tiles) * pairs)

    # ---- the step ------------------------------------------------------------
    def forward(self, ctx, xn, residual, cache) -> None:
        T, QH, KH, d = xn.shape[0], self.QH, self.KH, self.d
        g = cache.group
        fused = self.position.fused_rotary() if self.position is not None else (None, 0)
        slots = g.kv_slot if cache.write else None
        if fused is not None and d == 128 and fused[1] == d and fused[0] is not None and T > 256 and slots is not None and \
                xn.dtype == torch.bfloat16 and self.q_norm_w is not None and self.k_norm_w is not None:
            # a prompt portion with heads of 128: norm, rotation and the stores are the projection's own epilogue
            key = self.position.table_key()
            cs = ctx.shared.get(key)
            if cs is None:
                cs = ctx.shared[key] = ops.rope_table(ctx.positions, fused[0])
            q = torch.empty((T, QH, d), dtype=xn.dtype, device=xn.device)
            rows, scale = (xn.rows, xn.scale()) if isinstance(xn, RowScaled) else (xn, None)
            if ops.gemm_qkv_heads(rows, self.w_qkv, q, cache.kv, slots, cs, self.q_norm_w, self.k_norm_w, QH, KH, g.page_size, self.eps,
                                  row_scale=scale):
                attn = torch.empty((T, QH, d), dtype=xn.dtype, device=xn.device)
                ops.attention(ctx, q, cache.kv, g, attn, QH, KH, d, self.window or 0, self.scale)
                return matmul_into_residual(ctx, attn.view(T, QH * d), self.w_o, residual)
        if fused is not None and d == 128 and fused[1] == d and fused[0] is not None and 0 < T <= ops.STREAMING_TOKENS and \
                xn.dtype == torch.bfloat16 and (self.q_norm_w is None) == (self.k_norm_w is None):
            # a decode step's few rows with heads of 128: the cluster that reduces the projection does the per-head work
            rows, scale = (xn.rows, xn.scale()) if isinstance(xn, RowScaled) else (xn, None)
            q = torch.empty((T, QH, d), dtype=xn.dtype, device=xn.device)
            if ops.gemm_qkv_heads_stream(rows, self.w_qkv, q, cache.kv, slots, ctx.positions, fused[0], self.q_norm_w, self.k_norm_w,
                                         QH, KH, g.page_size, self.eps, row_scale=scale):
                attn = torch.empty((T, QH, d), dtype=xn.dtype, device=xn.device)
                ops.attention(ctx, q, cache.kv, g, attn, QH, KH, d, self.window or 0, self.scale)
                return matmul_into_residual(ctx, attn.view(T, QH * d), self.w_o, residual)
        qkv = matmul(ctx, xn, self.w_qkv)                                     # [T, (QH+2KH) d]; xn may be RowScaled
        act, dev = qkv.dtype, qkv.device
        q = torch.empty((T, QH, d), dtype=act, device=dev)
        if fused is not None:
            inv_freq, rot = fused
            cs = None
            if rot == d and d % 128 == 0 and act == torch.bfloat16 and inv_freq is not None and T > 64:
                # the angles depend on the step's positions only: for a large step the first layer tabulates
                # their cosines and sines (a small step computes them in place and saves the launch)
                key = self.position.table_key()          # equal for layers whose encodings make the same table
                cs = ctx.shared.get(key)
                if cs is None:
                    cs = ctx.shared[key] = ops.rope_table(ctx.positions, inv_freq)
            ops.qknorm_rope_append(qkv, self.q_norm_w, self.k_norm_w, inv_freq, ctx.positions, slots, q,
                                   cache.kv, QH, KH, d, rot, g.page_size, self.eps, cs_table=cs)
        else:
            # an encoding that is not a plain rotation: norm, then the part's own apply(), then append
            k = torch.empty((T, KH, d), dtype=act, device=dev)
            ops.qknorm_rope_append(qkv, self.q_norm_w, self.k_norm_w, None, None, None, q, None,
                                   QH, KH, d, 0, g.page_size, self.eps, k_out=k)
            self.position.apply(ctx, q, k, ctx.positions)
            if cache.write:
                ops.kv_append(k.view(T, KH * d), qkv[:, (QH + KH) * d:], g.kv_slot, cache.kv, KH, d, g.page_size)
        attn = torch.empty((T, QH, d), dtype=act, device=dev)
        ops.attention(ctx, q, cache.kv, g, attn, QH, KH, d, self.window or 0, self.scale)
        return matmul_into_residual(ctx, attn.view(T, QH * d), self.w_o, residual)


register_part("mixer", "attention", Attention)
