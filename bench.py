"""Throughput of the engine on one B200 at the three full-size shapes, random bf16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--shape 8b|4b|32b|<config.json>] [--batch 8]
                    [--context N] [--page-size 16] [--layers L] [--impl ours|reference] [--no-points]

Prints ONE JSON line.  By shape (reinfer_b200/shapes/*.json; the default is the 8B shape):
  8b   `value`: decoded tokens per second at --batch (8) and --context (4,096), the device alone: CUDA events
       around K replays of the captured decode step (every layer, the output head, the sampler), launched back to
       back.  `e2e`: the same K steps through the Python entry point (`LLM.step`: scheduler, the step's int32
       block from pinned memory to the device, the graph, sampled ids back to pinned memory) by the wall clock.
       `prefill`: one request of 2,048 tokens.  `roofline`: bytes the decode step has to read (every weight it
       uses once + the cache of the live requests) / its time, against the measured copy bandwidth.  `points`:
       decode at batch 1 and 64 (device and end to end) and batch 8 with pages of 64 tokens.
  4b   `value`: tokens per second (prompt + generated) over a run of 32 requests that arrive together, prompt lengths
       uniform in [128, 4096], prompts cut under a budget of 2,048 tokens a step beside the others' decode tokens;
       details under `mixed`; prefill, roofline (decode at --batch) and points as above.
  32b  as 8b at context 8,192; batch 64 runs to the longest context whose cache fits beside the weights
       (`points.b64_context`).
`segments`: where one eager step's time goes, by kernel family (us, TFLOP/s, GB/s); the table goes to stderr.
A decode step reads far more than the 126 MB L2 (16 GB of weights at the 8B shape), so no flush is made between
timed steps (config.l2 says so).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self):
        super().__init__(daemon=True)
        self.samples = []
        self.stop_flag = threading.Event()
        self.proc = None

    def run(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self.proc.stdout:
                self.samples.append([x.strip() for x in line.split(",")])
                if self.stop_flag.is_set():
                    break
        except OSError:
            pass

    def finish(self):
        self.stop_flag.set()
        if self.proc is not None:
            self.proc.terminate()
        self.join(timeout=2)
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(int(float(s[0])))
                mx = max(mx, int(float(s[1])))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


REFERENCE_UNAVAILABLE = ("the reference is a Rust workspace (no Python package, no cargo/rustc in this image): "
                         "pip cannot install it offline")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--shape", default="8b", help="8b, 4b, 32b or a config.json")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=None, help="tokens a request holds when the timed steps end")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--no-segments", action="store_true")
    a = ap.parse_args()
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)

    import torch
    from reinfer_b200 import measure, ops

    shape = a.shape.lower()
    big = shape.endswith("32b")
    mixed_run = shape.endswith("4b")
    ctx_len = a.context or (8192 if big else 4096)
    hbm_gbs, tf_burst, tf_sust, peak_src = measure.peaks(ROOT)
    page = a.page_size
    point_batches = [] if a.no_points else [1, 64]
    max_b = max([a.batch] + point_batches)
    if big:
        bench = measure.Bench(a.shape, layers=a.layers, page_size=page, max_num_seqs=max(max_b, 32) + 1, memory_fraction=0.9)
    else:
        need = max_b * (ctx_len + page) + 8192
        if mixed_run:
            need = max(need, 32 * (4096 + 128 + page))
        bench = measure.Bench(a.shape, layers=a.layers, page_size=page, pool_tokens=need, max_num_seqs=max(max_b, 32) + 1)
    eng = bench.engine
    pool_tokens = eng.cache.total_pages() * page

    prefill = bench.prefill(2048)
    prefill_out = {"value": prefill["value"], "tokens": 2048, "ms": prefill["ms"],
                   "frac": prefill["flops"] / (prefill["ms"] * 1e-3) / (tf_burst * 1e12), "peak": f"of {peak_src} burst"}

    def context_for(B):
        """The context that B requests can reach in this pool (each rounded up to pages, one page of head room)."""
        return min(ctx_len, (pool_tokens // B // page - 2) * page)

    clocks = ClockSampler()
    clocks.start()
    main_run = bench.decode(a.batch, a.steps, a.warmup, context_for(a.batch))
    clk = clocks.finish()
    points = {}
    for B in point_batches:
        c = context_for(B)
        r = bench.decode(B, max(8, a.steps // 4), 3, c)
        points[f"decode_b{B}"] = B / r["ms_device"] * 1e3
        points[f"e2e_b{B}"] = B / r["ms_e2e"] * 1e3
        points[f"roofline_b{B}"] = r["bytes"] / (r["ms_device"] * 1e-3) / 1e9 / hbm_gbs
        if c != ctx_len:
            points[f"b{B}_context"] = c
    mixed = None
    if mixed_run:
        mixed = bench.mixed(32, 128, 4096, 2048, 128, seed=0, passes=2)   # the second pass is reported
    seg = {}
    if not a.no_segments:
        for kind in ("decode", "prefill"):
            s = bench.segments(kind, B=a.batch, context=min(ctx_len, 4096))
            seg[kind] = measure.compact_segments(s)
            print(f"-- one eager {kind} step by segment (events; launches one after the other) --", file=sys.stderr)
            print("\n".join(measure.segment_table(s, hbm_gbs, tf_burst)), file=sys.stderr)
    status = ops.status_word()
    cfg, raw = bench.cfg, bench.raw
    h2d, d2h = main_run["h2d_bytes_per_step"], main_run["d2h_bytes_per_step"]
    layers, full_layers, load_s = bench.layers, bench.full_layers, bench.load_s
    wbytes = bench.weight_bytes
    if not a.no_points and not big and page != 64:
        # the same batch with pages of 64 tokens (one TMA box per 64-key tile instead of four)
        del bench, eng
        torch.cuda.empty_cache()
        b64 = measure.Bench(a.shape, layers=a.layers, page_size=64, pool_tokens=a.batch * (ctx_len + 64) + 8192,
                            max_num_seqs=a.batch + 1)
        r = b64.decode(a.batch, max(8, a.steps // 4), 3, ctx_len)
        points[f"decode_b{a.batch}_page64"] = a.batch / r["ms_device"] * 1e3

    ms_dev, ms_e2e = main_run["ms_device"], main_run["ms_e2e"]
    achieved = main_run["bytes"] / (ms_dev * 1e-3) / 1e9
    name = os.path.splitext(os.path.basename(measure.shape_path(a.shape)))[0]
    out = {
        "metric": f"decode tok/s ({name} shape, bf16, batch {a.batch}, context {main_run['context']})",
        "value": a.batch / ms_dev * 1e3, "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": ms_dev, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02) drawn on the device by the seeded generator, "
                                 "uniform-random token ids",
        "impl": "ours",
        "config": {"model": f"{name} shape", "layers": layers, "layers_of_model": full_layers,
                   "hidden": raw["hidden_size"], "q_heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
                   "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"],
                   "tied": bool(raw.get("tie_word_embeddings")), "global_batch": a.batch, "seq_len": main_run["context"],
                   "page_size": page, "parallelism": "single GPU",
                   "l2": "inputs (weights+cache per step) larger than L2, no flush", "sampling": "greedy on the GPU, in the step's graph"},
        "e2e": {"value": a.batch / ms_e2e * 1e3, "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": main_run["launches_per_step"] * a.steps,
        "prefill": prefill_out,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
                     "peak_source": f"of {peak_src}"},
        "points": points, "clocks": clk, "load_s": load_s, "kernel_status_word": status,
        "weight_gb": wbytes / 1e9,
    }
    if mixed is not None:
        out["metric"] = (f"tokens/s (prompt + generated) of 32 requests arriving together, prompts 128-4096, budget 2048 "
                         f"a step ({name} shape, bf16)")
        out["decode"] = {"value": out["value"], "ms_per_step": ms_dev, "batch": a.batch, "context": main_run["context"]}
        out["value"] = mixed["tokens_per_s"]
        out["ms_per_step"] = mixed["seconds"] / mixed["steps"] * 1e3
        out["steps"] = mixed["steps"]
        out["mixed"] = mixed
        out["e2e"]["note"] = "decode at --batch through LLM.step; the mixed run itself is end to end (value)"
    if seg:
        out["segments"] = seg
    print(json.dumps(out))
    return 0 if status == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
