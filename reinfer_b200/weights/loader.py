"""Binding tensors of a model folder to the names that the model's parts declare.

Rule of storage: a floating tensor stored in 16 bits is kept as bfloat16 (float16
is converted once), one stored in 32 bits stays 32-bit, integer tables become
int32.  With `compute_dtype=torch.float32` every floating tensor is widened to
float32 instead, so that the 32-bit path sees no rounding of its own.  The
reference converts everything to f16 and transposes (crates/cuda/src/engine.rs:
6523-6598); neither is done here: matrices stay `[out, in]` as stored.

All mismatches are collected and reported in ONE error that lists missing
tensors, unexpected tensors and wrong shapes (the reference stops at the first,
engine.rs:3213-3224).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, Mapping, Optional, Set

import torch

from .params import ParamSpec
from .safetensors_io import open_model_tensors, write_safetensors


class WeightError(ValueError):
    """One error for everything that is wrong between a file and a model."""

    def __init__(self, where: str, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        self.wrong_dtype = sorted(wrong_dtype)
        lines = [f"{where}: the tensors do not fit the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: expected {list(e)} got {list(g)}" for n, e, g in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtype ({len(self.wrong_dtype)}): " + "; ".join(
                f"{n}: {why}" for n, why in self.wrong_dtype))
        super().__init__("\n".join(lines))


def _convert(t: torch.Tensor, spec: ParamSpec, compute_dtype: torch.dtype) -> torch.Tensor:
    if spec.kind == "int":
        return t.to(torch.int32)
    if compute_dtype == torch.float32:
        return t.to(torch.float32)
    if t.dtype in (torch.float32, torch.float64):
        return t.to(torch.float32)
    return t.to(torch.bfloat16)


def load_state(model_dir: str, expected: Mapping[str, ParamSpec], compute_dtype: torch.dtype,
               device, ignorable: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """Read every expected tensor of `model_dir`, check names, shapes and kinds,
    convert by the storage rule and move to `device`."""
    found = open_model_tensors(model_dir)
    ignorable = set(ignorable)
    missing, wrong_shape, wrong_dtype = [], [], []
    for name, spec in expected.items():
        if name not in found:
            if not spec.optional:
                missing.append(name)
            continue
        f, n = found[name]
        if tuple(f.shape(n)) != tuple(spec.shape):
            wrong_shape.append((name, tuple(spec.shape), tuple(f.shape(n))))
        is_float = f.dtype(n).is_floating_point
        if spec.kind == "int" and is_float:
            wrong_dtype.append((name, f"expected an integer table, stored as {f.dtype(n)}"))
        if spec.kind == "float" and not is_float:
            wrong_dtype.append((name, f"expected floating point, stored as {f.dtype(n)}"))
    unexpected = [n for n in found if n not in expected and n not in ignorable]
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(model_dir, missing, unexpected, wrong_shape, wrong_dtype)
    out: Dict[str, torch.Tensor] = {}
    for name, spec in expected.items():
        if name not in found:
            continue
        f, n = found[name]
        t = f.tensor(n)
        if device is not None and str(device) != "cpu":
            # upload in the stored width, convert on the device (one pass over PCIe)
            out[name] = _convert(t.to(device, non_blocking=False), spec, compute_dtype).contiguous()
        else:
            out[name] = _convert(t, spec, compute_dtype).contiguous().clone()
    return out


def random_state(expected: Mapping[str, ParamSpec], seed: int, dtype: torch.dtype,
                 device="cpu") -> Dict[str, torch.Tensor]:
    """Seeded random tensors for every expected name: matrices and
    tables N(0, std), norm weights 1 + N(0, 0.05), integer tables 15-bit uniform.
    Every element is a fixed function of (seed, tensor name, its row-major index)
    (weights/random.py), so a tensor's values depend neither on which other
    tensors exist nor on where they are drawn: a model drawn on the GPU and one
    written to a folder on the CPU hold the same numbers.  Values are float32,
    rounded to `dtype`."""
    from . import random as rnd
    out: Dict[str, torch.Tensor] = {}
    dev = torch.device(device)
    for name, spec in expected.items():
        # (a tensor that a file may lack is drawn too: a random untied model has an output matrix of its own)
        if spec.kind == "int":
            out[name] = rnd.ints(spec.shape, seed, name, dev)
        elif spec.init == "zeros":
            out[name] = torch.zeros(spec.shape, dtype=dtype, device=dev)
        elif spec.init == "norm":
            out[name] = rnd.normal(spec.shape, seed, name, 1.0, 0.05, dtype, dev)
        else:
            out[name] = rnd.normal(spec.shape, seed, name, 0.0, spec.std, dtype, dev)
    return out


def write_random_model(model_dir: str, config, seed: int, dtype: torch.dtype = torch.float32) -> str:
    """Random-weights mode: write `config.json` and `model.safetensors` for `config`
    (a typed configuration of a registered architecture) and return the folder."""
    from ..config.registry import resolve_architecture
    from ..parts.model import expected_params
    raw = config.to_dict()
    arch = resolve_architecture(raw)
    spec = arch.build_spec(config)
    expected = expected_params(spec)
    state = random_state(expected, seed, dtype, "cpu")
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(raw, f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), state,
                      metadata={"format": "pt", "seed": seed})
    return model_dir
