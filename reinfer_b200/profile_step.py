"""A few steps of a random-weight model for a profiler to look at:

    python -m reinfer_b200.profile_step --mode decode|prefill|timeline|gemm-tiles [--shape qwen3-8b|4b|32b|<config.json>]
                                        --batch B --context N [--layers L] [--steps K] [--page-size P]

builds a random-weight model of the shape (reinfer_b200/shapes/, or fewer layers of it), fills B requests to N tokens, runs two
warm-up steps, and brackets K steps of the chosen kind with cudaProfilerStart/Stop, so that
`ncu --profile-from-start off` sees exactly those (the reference brackets its step with event
profilers instead, crates/cuda/src/engine.rs:928-1408).  Decode steps are launched eagerly
(no graph), so every kernel appears as its own launch.

`--mode timeline` needs no profiler: it builds the kernels with -DRB_TIMELINE (every CTA records its start, the
moment its wait for the kernels before it returned, and its end, by the global timer), replays ONE decode step
through the CUDA graph as serving does - with programmatic dependent launch, so kernels overlap - after a
flush of L2, and prints for every launch when its first CTA started, when its wait returned, when its last CTA
ended, and by how much it moved the end of the step.

`--mode gemm-tiles` (the same build flag) runs the four products of one layer of the shape over --prefill-tokens
tokens and prints, for every tile a persistent CTA walks, what its issuing threads did: how long the tile's products
took to issue, how long the issuing thread waited for operands, the producer for free stages, and the epilogue's span.
"""
from __future__ import annotations

import argparse
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--mode", choices=["decode", "prefill", "timeline", "gemm-tiles"], default="decode")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4000)
    ap.add_argument("--shape", default="qwen3-8b", help="a file of reinfer_b200/shapes (qwen3-8b, 4b, 32b) or a config.json")
    ap.add_argument("--layers", type=int, default=None, help="build only this many layers of the shape")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    a = ap.parse_args(argv)

    if a.mode in ("timeline", "gemm-tiles"):
        from .csrc import build                   # the flag is part of the build key: a library of its own
        if "-DRB_TIMELINE" not in build.FLAGS:
            build.FLAGS.append("-DRB_TIMELINE")
    import torch
    from . import measure, ops
    from .engine import Engine, StepEntry

    _raw, cfg, _full = measure.load_shape(a.shape, a.layers)
    a.layers = int(_raw["num_hidden_layers"])
    if a.mode == "gemm-tiles":
        return gemm_tiles(ops, torch, _raw, a.prefill_tokens)
    B, N = a.batch, a.context
    eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", page_size=a.page_size,
                             max_tokens=B * (N + a.page_size) + 2 * a.prefill_tokens, max_num_seqs=B + 1,
                             cuda_graphs=a.mode == "timeline")
    g = torch.Generator().manual_seed(0)
    for b in range(B):
        toks = torch.randint(0, cfg.vocab_size, (N,), generator=g).tolist()
        for i in range(0, N, 2048):
            eng.step([StepEntry(b, toks[i:i + 2048], [])])

    def decode():
        return eng.step([StepEntry(b, [5 + b], [0]) for b in range(B)])

    for _ in range(4 if a.mode == "timeline" else 2):
        decode()
    torch.cuda.synchronize()
    if a.mode == "timeline":
        return timeline(ops, torch, decode, B, N, a.layers)
    torch.cuda.profiler.start()
    for k in range(a.steps):
        if a.mode == "decode":
            decode()
        else:
            toks = torch.randint(0, cfg.vocab_size, (a.prefill_tokens,), generator=g).tolist()
            eng.step([StepEntry(f"p{k}", toks, [a.prefill_tokens - 1])])
            eng.finish(f"p{k}")
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    err = ops.kernel_error()
    print(f"profiled {a.steps} {a.mode} steps, batch {B}, context {N}, layers {a.layers}; kernel error word {err}")
    return 0 if err == 0 else 1


def gemm_tiles(ops, torch, raw, T: int) -> int:
    """The tile trace of the persistent products (gemm_tc.cu, rb_gemm_tile_trace): ten words per CTA and tile."""
    import ctypes
    lib = ops.lib()
    if not hasattr(lib, "rb_gemm_tile_trace"):
        print("the library was not built with -DRB_TIMELINE")
        return 1
    h, F = int(raw["hidden_size"]), int(raw["intermediate_size"])
    qkv = (int(raw["num_attention_heads"]) + 2 * int(raw["num_key_value_heads"])) * int(raw["head_dim"])
    o_in = int(raw["num_attention_heads"]) * int(raw["head_dim"])
    CAP, W, dev = 16, 10, "cuda"
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    print(f"tiles of the four products of a layer over {T} tokens; per local tile of a CTA (mean over the CTAs that have it):")
    print("  product          tile  ctas  begin us  span us  k-step ns  SM MHz  issue clk/k  commit clk/k  wait operands clk/k  "
          "producer waits clk/k  epilogue us  drained at us")
    for name, N, K, kind in (("qkv", qkv, h, "store"), ("o", h, o_in, "add"), ("gate/up", F, h, "swiglu"), ("down", h, F, "add")):
        x = (torch.randn(T, K, device=dev) * 0.1).bfloat16()
        ws = [(torch.randn(2 * N if kind == "swiglu" else N, K, device=dev) * 0.02).bfloat16() for _ in range(4)]
        c = torch.zeros(T, N, device=dev, dtype=torch.float32 if kind == "add" else torch.bfloat16)
        go = (lambda w: ops.gemm_bf16_swiglu(x, w, c)) if kind == "swiglu" else (lambda w: ops.gemm_bf16(x, w, c, accumulate=kind == "add"))
        for w in ws[:3]:
            go(w)
        torch.cuda.synchronize()
        buf = torch.zeros(sms * CAP * W, dtype=torch.int64, device=dev)
        lib.rb_gemm_tile_trace(ctypes.c_void_p(buf.data_ptr()), ctypes.c_int(CAP))
        go(ws[3])
        torch.cuda.synchronize()
        lib.rb_gemm_tile_trace(ctypes.c_void_p(0), ctypes.c_int(0))
        b = buf.cpu().view(sms, CAP, W).double()
        nkb = -(-K // 64)
        started = b[:, :, 6][b[:, :, 6] > 0]
        if started.numel() == 0:
            print(f"  {name}: no records (the product did not take the persistent kernel)")
            continue
        t0 = started.min()
        for l in range(CAP):
            m = b[:, l, 0] > 0
            if not m.any():
                break
            f = lambda i: b[:, l, i][m]
            span = f(2) - f(0)
            print(f"  {name + ' ' + str(N) + 'x' + str(K):16s} {l:4d} {int(m.sum()):5d} {((f(0) - t0) / 1e3).mean():9.2f} {(span / 1e3).mean():8.2f} "
                  f"{(span / nkb).mean():10.1f} {(f(8) / span * 1e3).mean():7.0f} {(f(9) / nkb).mean():12.0f} {(f(3) / nkb).mean():13.0f} "
                  f"{(f(1) / nkb).mean():20.0f} {(f(7) / nkb).mean():21.0f} {((f(5) - f(4)) / 1e3).mean():12.2f} {((f(5) - t0) / 1e3).max():14.2f}")
    err = ops.kernel_error()
    return 0 if err == 0 else 1


TIMELINE_NAMES = {2: "norm", 3: "qknorm_rope", 4: "fa_decode", 5: "merge", 6: "gemm", 7: "gemm_gated", 8: "gemm_persist",
                  9: "gemm_gated_p", 10: "fa_prefill"}
TIMELINE_SETTERS = ("rb_gemm_step_timeline", "rb_attn_step_timeline", "rb_elementwise_step_timeline")


def timeline(ops, torch, decode, B, N, layers) -> int:
    import ctypes
    lib = ops.lib()
    cap = 1 << 18
    buf = torch.zeros(4 + cap * 4, dtype=torch.int64, device="cuda")
    buf[1] = cap
    flush = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")
    flush.zero_()
    torch.cuda.synchronize()
    for fn in TIMELINE_SETTERS:
        getattr(lib, fn)(ctypes.c_void_p(buf.data_ptr()))
    # the decode attention's own stamps: eight per CTA, every launch writes over the one before, so the last layer's stay
    phases = torch.zeros(8192 * 8, dtype=torch.int64, device="cuda") if hasattr(lib, "rb_fa_decode_trace") else None
    if phases is not None:
        lib.rb_fa_decode_trace(ctypes.c_void_p(phases.data_ptr()))
    decode()
    torch.cuda.synchronize()
    for fn in TIMELINE_SETTERS:
        getattr(lib, fn)(ctypes.c_void_p(0))
    if phases is not None:
        lib.rb_fa_decode_trace(ctypes.c_void_p(0))
    h = buf.cpu()
    n = min(int(h[0]), cap)
    rec = h[4:4 + n * 4].view(-1, 4)
    ids, st, en, mk = (rec[:, 0] >> 32).tolist(), rec[:, 1].tolist(), rec[:, 2].tolist(), rec[:, 3].tolist()
    blk = (rec[:, 0] & 0xFFFFFFFF).tolist()
    # CTAs of one launch: a run (by start time) of records of one kernel whose starts lie before the run's end; a block
    # index that the run has already seen begins the next launch of the same kernel (the device hands out a launch's
    # CTAs only when all of the launch before it have been handed out)
    launches = []
    for i in sorted(range(n), key=lambda j: st[j]):
        m = mk[i] or 1 << 62
        if launches and launches[-1]["id"] == ids[i] and st[i] < launches[-1]["end"] + 200 and blk[i] not in launches[-1]["blocks"]:
            l = launches[-1]
            l["end"] = max(l["end"], en[i]); l["n"] += 1; l["mark"] = min(l["mark"], m); l["blocks"].add(blk[i])
        else:
            launches.append(dict(id=ids[i], start=st[i], end=en[i], n=1, mark=m, blocks={blk[i]}))
    if not launches:
        print("no records: the library was not built with -DRB_TIMELINE")
        return 1
    t0 = launches[0]["start"]
    print(f"one decode step by graph replay: batch {B}, context {N}, {layers} layers; {n} CTAs in {len(launches)} launches; us since the first CTA")
    print(f"{'kernel':12s} {'ctas':>5s} {'start':>9s} {'waited':>9s} {'end':>9s} {'moved the end by':>17s}")
    prev_end, tot = t0, {}
    for l in launches:
        name = TIMELINE_NAMES.get(l["id"], str(l["id"]))
        adv = max(0, l["end"] - prev_end)
        prev_end = max(prev_end, l["end"])
        tot[name] = tot.get(name, 0) + adv
        waited = (l["mark"] - t0) / 1e3 if l["mark"] < 1 << 62 else float("nan")
        print(f"{name:12s} {l['n']:5d} {(l['start'] - t0) / 1e3:9.2f} {waited:9.2f} {(l['end'] - t0) / 1e3:9.2f} {adv / 1e3:17.2f}")
    print("the step's end moved, by kernel (us):", {k: round(v / 1e3, 1) for k, v in tot.items()}, "total", round((prev_end - t0) / 1e3, 1))
    if phases is not None:
        t = phases.view(-1, 8).cpu()
        t = t[t[:, 0] > 0]
        if t.shape[0]:
            first = t[:, 0].min()
            rel = (t - first).double() / 1e3
            rel[t == 0] = float("nan")
            print(f"decode attention of the last layer, {t.shape[0]} CTAs, us since its first CTA began (mean / min / max over the CTAs):")
            for i, name in enumerate(("began", "shared memory zeroed", "kernels before done", "first tile landed", "last tile used",
                                      "own part sent", "cluster barrier passed", "end")):
                col = rel[:, i]
                col = col[~torch.isnan(col)]
                if col.numel():
                    print(f"   {name:22s} {col.mean().item():7.2f} {col.min().item():7.2f} {col.max().item():7.2f}")
    err = ops.kernel_error()
    return 0 if err == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
