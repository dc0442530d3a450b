"""Seeded random tensors from a counter: element `i` of tensor `name` under `seed` is one
fixed function of (seed, name, i), so the same values come out on the CPU and on the GPU,
in any order, in pieces, and without a file.  The reference has no random-weights mode;
the mixing function and its constants are its SplitMix64 (crates/scheduler/src/rng.rs:
12-30), which the sampler uses too.

    base   = splitmix64(seed ^ fnv1a64(name))          splitmix64(x) = mix(x + GOLDEN)
    a, b   = mix(base + (2i+1) GOLDEN), mix(base + (2i+2) GOLDEN)     (outputs 2i+1 and 2i+2 of
                                                        the SplitMix64 stream that starts at base)
    u1, u2 = ((a >> 11) + 1) / 2^53 in (0, 1],  (b >> 11) / 2^53 in [0, 1)
    value  = float32( mean + std * sqrt(-2 ln u1) * cos(2 pi u2) )    Box-Muller in float64,
             every operation rounded on its own (no fused multiply-add)
    integer tables:  a >> 49  (15 bits)

The float64 logarithm and cosine of the CPU's and the GPU's libraries may differ in their
last bit; after the rounding to float32 that shows in about one element of 10^8, by one
unit in the last place.
"""
from __future__ import annotations

from typing import Sequence

import torch

_M64 = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15
_C1, _C2 = 0xBF58476D1CE4E5B9, 0x94D049BB133111EB
TWO_PI = 6.283185307179586
_CHUNK = 1 << 20


def _mix(z: int) -> int:
    z = ((z ^ (z >> 30)) * _C1) & _M64
    z = ((z ^ (z >> 27)) * _C2) & _M64
    return z ^ (z >> 31)


def fnv1a64(text: str) -> int:
    h = 0xCBF29CE484222325
    for byte in text.encode("utf-8"):
        h = ((h ^ byte) * 0x100000001B3) & _M64
    return h


def stream_base(seed: int, name: str) -> int:
    """Where the tensor's stream starts: splitmix64(seed ^ fnv1a64(name))."""
    return _mix((((int(seed) & _M64) ^ fnv1a64(name)) + GOLDEN) & _M64)


def _signed(v: int) -> int:
    v &= _M64
    return v - (1 << 64) if v >= (1 << 63) else v


def _mix_i64(z: torch.Tensor) -> torch.Tensor:
    """mix() on int64 tensors: products wrap like unsigned ones, shifts are made logical by masking."""
    z = (z ^ ((z >> 30) & ((1 << 34) - 1))) * _signed(_C1)
    z = (z ^ ((z >> 27) & ((1 << 37) - 1))) * _signed(_C2)
    return z ^ ((z >> 31) & ((1 << 33) - 1))


def _draws(base: int, start: int, stop: int):
    k = torch.arange(start, stop, dtype=torch.int64) * _signed(2 * GOLDEN)
    return _mix_i64(k + _signed(base + GOLDEN)), _mix_i64(k + _signed(base + 2 * GOLDEN))


def normal_cpu(shape: Sequence[int], base: int, mean: float, std: float) -> torch.Tensor:
    """float32 tensor of `shape` on the CPU, element i (row-major) as the module's formula says."""
    n = 1
    for s in shape:
        n *= int(s)
    out = torch.empty(n, dtype=torch.float32)
    for start in range(0, n, _CHUNK):
        stop = min(n, start + _CHUNK)
        a, b = _draws(base, start, stop)
        u1 = (((a >> 11) & ((1 << 53) - 1)).double() + 1.0) * 2.0 ** -53
        u2 = ((b >> 11) & ((1 << 53) - 1)).double() * 2.0 ** -53
        x = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(TWO_PI * u2)
        out[start:stop] = (x * float(std) + float(mean)).float()
    return out.reshape(tuple(shape))


def ints_cpu(shape: Sequence[int], base: int) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= int(s)
    out = torch.empty(n, dtype=torch.int32)
    for start in range(0, n, _CHUNK):
        stop = min(n, start + _CHUNK)
        a, _ = _draws(base, start, stop)
        out[start:stop] = ((a >> 49) & 0x7FFF).int()
    return out.reshape(tuple(shape))


def normal(shape: Sequence[int], seed: int, name: str, mean: float, std: float, dtype: torch.dtype,
           device) -> torch.Tensor:
    """The tensor `name` of a random model: drawn by the kernel on a CUDA device, by torch's integer
    arithmetic on the CPU; float32 values rounded to `dtype` (round to nearest even) either way."""
    base = stream_base(seed, name)
    dev = torch.device(device)
    if dev.type == "cuda":
        from .. import ops
        out = torch.empty(tuple(shape), dtype=dtype, device=dev)
        ops.random_normal(out, base, mean, std)
        return out
    return normal_cpu(shape, base, mean, std).to(dtype)


def ints(shape: Sequence[int], seed: int, name: str, device) -> torch.Tensor:
    base = stream_base(seed, name)
    dev = torch.device(device)
    if dev.type == "cuda":
        from .. import ops
        out = torch.empty(tuple(shape), dtype=torch.int32, device=dev)
        ops.random_ints(out, base)
        return out
    return ints_cpu(shape, base)
