#!/usr/bin/env python3
"""Golden vectors from the reference's own kernels.

The reference (LeonRust/reinfer) is a Rust workspace and cannot be built here, but its CUDA kernels are
plain `extern "C" __global__` functions in self-contained files (crates/cuda/kernels/*.cu).  This script
compiles four of those files UNCHANGED with nvcc - each is #included from a few lines of launcher code
written below, nothing of the reference is copied into this repository - runs them on a GPU on small
seeded inputs, and writes inputs and outputs to `reference_kernels.json` beside this file.  The tests
(tests/test_golden.py on the CPU, tests/test_golden_gpu.py on the GPU) hold the plain implementation and
this engine's kernels against those numbers: a reading error shared by the engine and the plain
implementation (the order of head norm and rotation, the pairing of the rotation, where eps sits, the
SplitMix64 and Gumbel constants, the filters' order) would show there.

    python tests/golden/make_golden.py --reference /path/to/reinfer [--out tests/golden/reference_kernels.json]

Kernels run (file:line of the reference): diff_kernels.cu:7 rms_norm_row, :26 rope_row, :157 masked_softmax_row;
dense_kernels.cu:92 rms_norm_heads_f16, :152 rope_heads_f16, :202 swiglu_f16, :363 swiglu_f32;
decode_gqa_kernels.cu:69 decode_step_gqa; sampler_kernel.cu:155 gpu_sampler_kernel.
It needs a CUDA device and nvcc; the committed JSON is what the tests read.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

LAUNCHERS = {
    "diff": ('#include "diff_kernels.cu"\n'
             'extern "C" void g_rms_norm_row(const float* x, const float* w, float* o, int n, float eps) { rms_norm_row<<<1, 256>>>(x, w, o, n, eps); }\n'
             'extern "C" void g_rope_row(const float* x, float* o, int half, int pos, float eta) { rope_row<<<1, 1024>>>(x, o, half, pos, eta); }\n'
             'extern "C" void g_masked_softmax_row(const float* x, float* o, int n) { masked_softmax_row<<<1, 256>>>(x, o, n); }\n'),
    "dense": ('#include "dense_kernels.cu"\n'
              'extern "C" void g_rms_norm_heads_f16(const unsigned short* x, unsigned short* o, const unsigned short* w, int rows, int n, float eps) { rms_norm_heads_f16<<<rows, 256>>>(x, o, w, rows, n, eps); }\n'
              'extern "C" void g_rope_heads_f16(unsigned short* x, int heads, int half, int pos, float eta, float scale) { rope_heads_f16<<<heads, 1024>>>(x, heads, half, pos, eta, scale); }\n'
              'extern "C" void g_swiglu_f16(const unsigned short* g, const unsigned short* u, unsigned short* o, int n) { swiglu_f16<<<(n + 255) / 256, 256>>>(g, u, o, n); }\n'
              'extern "C" void g_swiglu_f32(const float* g, const float* u, float* o, int n) { swiglu_f32<<<(n + 255) / 256, 256>>>(g, u, o, n); }\n'),
    "gqa": ('#include "decode_gqa_kernels.cu"\n'
            'extern "C" void g_decode_step_gqa(const unsigned short* q, const unsigned int* page, const unsigned short* kv, const unsigned int* lens,\n'
            '    float* scores, unsigned short* out, int B, int QH, int d, int block_len, int kv_ratio, int kv_heads, int max_kv, int total_pages) {\n'
            '    decode_step_gqa<<<B * QH, 256>>>(q, page, kv, lens, scores, out, B, QH, d, block_len, kv_ratio, kv_heads, max_kv, total_pages); }\n'),
    "sampler": ('#include "sampler_kernel.cu"\n'
                'extern "C" void g_sampler(const float* logits, const unsigned* window, unsigned window_len, const unsigned* bias_ids, const float* bias_vals,\n'
                '    unsigned n_bias, float freq, float pres, float rep, float temp, unsigned top_k, float top_p, float min_p, unsigned long long base,\n'
                '    unsigned vocab, float* val, float* prob, unsigned* out) {\n'
                '    gpu_sampler_kernel<<<1, 256>>>(logits, window, window_len, bias_ids, bias_vals, n_bias, freq, pres, rep, temp, top_k, top_p, min_p, base, vocab, val, prob, out); }\n'),
}

M64 = (1 << 64) - 1


def mix(z):
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
    return z ^ (z >> 31)


def stream_output(seed, n):
    """The n-th (1-based) output of SplitMix64::new(seed) (crates/scheduler/src/rng.rs:36-50): what the host hands the
    sampler kernel as `rng_base` at the request's n-th draw (crates/cuda/src/sampler.rs:220)."""
    return mix((seed + n * 0x9E3779B97F4A7C15) & M64)


def build(reference: str, workdir: str) -> ctypes.CDLL:
    kernels = os.path.join(reference, "crates", "cuda", "kernels")
    objs = []
    for name, text in LAUNCHERS.items():
        src = os.path.join(workdir, f"launch_{name}.cu")
        with open(src, "w") as f:
            f.write(text)
        obj = src[:-3] + ".o"
        subprocess.run(["nvcc", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-I", kernels,
                        "-c", src, "-o", obj], check=True)
        objs.append(obj)
    lib = os.path.join(workdir, "libgolden.so")
    subprocess.run(["nvcc", "-shared", "-o", lib] + objs, check=True)
    return ctypes.CDLL(lib)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="a checkout of LeonRust/reinfer")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_kernels.json"))
    a = ap.parse_args()
    import torch
    rng = np.random.RandomState(20251)
    dev = "cuda"
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    f32 = lambda arr: torch.tensor(np.asarray(arr, dtype=np.float32), device=dev)
    f16bits = lambda arr: torch.tensor(np.asarray(arr, dtype=np.float16).view(np.uint16).astype(np.int32), device=dev).to(torch.int16)
    bits_of = lambda t: (t.cpu().numpy().view(np.uint16)).astype(int).tolist()
    cases = {}
    with tempfile.TemporaryDirectory() as wd:
        lib = build(a.reference, wd)
        # ---- RMSNorm, float32
        out = []
        for n, eps in ((96, 1e-5), (64, 1e-6), (200, 1e-4)):
            x, w = rng.randn(n) * 1.7, 1 + 0.05 * rng.randn(n)
            xd, wd_, od = f32(x), f32(w), torch.zeros(n, device=dev)
            lib.g_rms_norm_row(P(xd), P(wd_), P(od), n, ctypes.c_float(eps))
            out.append({"n": n, "eps": eps, "x": xd.tolist(), "w": wd_.tolist(), "out": od.tolist()})
        cases["rms_norm_row"] = out
        # ---- rotation, float32
        out = []
        for half, pos, eta in ((16, 0, 1e6), (16, 1, 1e6), (16, 37, 1e6), (8, 1000, 1e4), (64, 513, 1e6)):
            x = rng.randn(2 * half)
            xd, od = f32(x), torch.zeros(2 * half, device=dev)
            lib.g_rope_row(P(xd), P(od), half, pos, ctypes.c_float(eta))
            out.append({"half": half, "pos": pos, "eta": eta, "x": xd.tolist(), "out": od.tolist()})
        cases["rope_row"] = out
        # ---- softmax over a row with masked places
        x = rng.randn(50) * 3
        x[[3, 17, 49]] = -np.inf
        xd, od = f32(x), torch.zeros(50, device=dev)
        lib.g_masked_softmax_row(P(xd), P(od), 50)
        cases["masked_softmax_row"] = [{"x": [v if np.isfinite(v) else "-inf" for v in xd.tolist()], "out": od.tolist()}]
        # ---- per-head RMSNorm then rotation, float16 storage (the order of crates/cuda/src/engine.rs:4122-4160)
        rows, n, eps, pos, eta = 6, 32, 1e-6, 37, 1e6
        x, w = rng.randn(rows, n), 1 + 0.05 * rng.randn(n)
        xd, wd_, od = f16bits(x), f16bits(w), torch.zeros(rows, n, dtype=torch.int16, device=dev)
        lib.g_rms_norm_heads_f16(P(xd), P(od), P(wd_), rows, n, ctypes.c_float(eps))
        normed = bits_of(od)
        lib.g_rope_heads_f16(P(od), rows, n // 2, pos, ctypes.c_float(eta), ctypes.c_float(1.0))
        cases["head_norm_then_rope_f16"] = [{"rows": rows, "n": n, "eps": eps, "pos": pos, "eta": eta, "x_bits": bits_of(xd),
                                             "w_bits": bits_of(wd_), "normed_bits": normed, "out_bits": bits_of(od)}]
        # ---- SwiGLU
        g, u = rng.randn(77) * 3, rng.randn(77)
        gd, ud, od = f32(g), f32(u), torch.zeros(77, device=dev)
        lib.g_swiglu_f32(P(gd), P(ud), P(od), 77)
        g16, u16, o16 = f16bits(g), f16bits(u), torch.zeros(77, dtype=torch.int16, device=dev)
        lib.g_swiglu_f16(P(g16), P(u16), P(o16), 77)
        cases["swiglu"] = [{"gate": gd.tolist(), "up": ud.tolist(), "out": od.tolist(), "gate_bits": bits_of(g16), "up_bits": bits_of(u16),
                            "out_bits": bits_of(o16)}]
        # ---- decode attention over a paged cache, grouped heads (q comes scaled by 1/sqrt(d), engine.rs:4150-4160)
        QH, KH, d, BL, kv_len, total_pages = 6, 2, 32, 8, 21, 5
        pages = [3, 0, 4]
        q = rng.randn(QH, d) / np.sqrt(d)
        k, v = rng.randn(kv_len, KH, d), rng.randn(kv_len, KH, d)
        kv = np.zeros((2, total_pages, BL, KH, d))
        for t in range(kv_len):
            kv[0, pages[t // BL], t % BL], kv[1, pages[t // BL], t % BL] = k[t], v[t]
        qd, kvd = f16bits(q), f16bits(kv)
        paged = torch.tensor(pages, dtype=torch.int32, device=dev)
        lens = torch.tensor([kv_len], dtype=torch.int32, device=dev)
        scores = torch.zeros(QH * 32, device=dev)
        od = torch.zeros(QH, d, dtype=torch.int16, device=dev)
        lib.g_decode_step_gqa(P(qd), P(paged), P(kvd), P(lens), P(scores), P(od), 1, QH, d, BL, QH // KH, KH, 32, total_pages)
        cases["decode_step_gqa"] = [{"QH": QH, "KH": KH, "d": d, "kv_len": kv_len, "q_scaled_bits": bits_of(qd),
                                     "k_bits": bits_of(f16bits(k)), "v_bits": bits_of(f16bits(v)), "out_bits": bits_of(od)}]
        # ---- the sampler: one launch per (parameters, seed, draw)
        vocab = 500
        out = []
        logits = rng.randn(vocab) * 2.5
        logits[[11, 300]] = [np.nan, -np.inf]
        ld = f32(logits)
        val, prob = torch.zeros(vocab, device=dev), torch.zeros(vocab, device=dev)
        res = torch.zeros(3, dtype=torch.int32, device=dev)
        settings = [dict(temperature=0.0), dict(temperature=0.8), dict(temperature=1.3, top_k=10), dict(temperature=1.0, top_p=0.9),
                    dict(temperature=1.0, min_p=0.1), dict(temperature=0.7, top_k=40, top_p=0.8, min_p=0.02),
                    dict(temperature=0.0, rep=1.5, window=[int(np.nanargmax(np.where(np.isfinite(logits), logits, -1e9))), 7, 7]),
                    dict(temperature=0.9, freq=0.3, pres=0.4, window=[5, 9, 9, 120, 5, 9]),
                    dict(temperature=0.6, bias=[(3, 4.0), (77, -2.5), (450, 1.0)])]
        for s in settings:
            for seed, draw in ((1, 1), (1, 2), (12345678901234567, 40)):
                window = torch.tensor(s.get("window", [0]), dtype=torch.int32, device=dev)
                bias = sorted(s.get("bias", []))
                bids = torch.tensor([b[0] for b in bias] or [0], dtype=torch.int32, device=dev)
                bvals = f32([b[1] for b in bias] or [0.0])
                base = stream_output(seed, draw)
                res.zero_()
                lib.g_sampler(P(ld), P(window), len(s.get("window", [])), P(bids), P(bvals), len(bias),
                              ctypes.c_float(s.get("freq", 0.0)), ctypes.c_float(s.get("pres", 0.0)), ctypes.c_float(s.get("rep", 1.0)),
                              ctypes.c_float(s["temperature"]), s.get("top_k", 0), ctypes.c_float(s.get("top_p", 1.0)),
                              ctypes.c_float(s.get("min_p", 0.0)), ctypes.c_ulonglong(base), vocab, P(val), P(prob), P(res))
                torch.cuda.synchronize()
                token, _tie, status = res.tolist()
                out.append({"settings": s, "seed": seed, "draw": draw, "rng_base": str(base), "token": token, "status": status})
        cases["gpu_sampler_kernel"] = {"logits": [v if np.isfinite(v) else str(v) for v in ld.tolist()], "draws": out}
        torch.cuda.synchronize()
    head = {"made_by": "tests/golden/make_golden.py", "reference": "LeonRust/reinfer, crates/cuda/kernels (compiled unchanged)",
            "device": torch.cuda.get_device_name(0)}
    with open(a.out, "w") as f:
        json.dump({"header": head, "cases": cases}, f)
    print(f"wrote {a.out}: {os.path.getsize(a.out)} bytes, {sum(len(c) if isinstance(c, list) else len(c['draws']) for c in cases.values())} cases")
    return 0


if __name__ == "__main__":
    sys.exit(main())
