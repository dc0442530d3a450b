"""Decode and prefill throughput of the Qwen3-8B shape on one B200, random bf16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096]
                    [--layers L] [--impl ours|reference]

Prints ONE JSON line.  `value`: decoded tokens per second at the given batch, timed on the
device alone: CUDA events around K decode steps launched back to back (the step's captured graph
- every layer, the output head - and the sampler kernel), no host work in between.  `e2e`: K more
steps of the same requests through the Python entry point (`LLM.step`: scheduler, the step's int32
block from pinned memory to the device, the graph, the sampler, sampled ids back to pinned
memory), by the wall clock.  `prefill`:
one request of 2,048 tokens.  `roofline`: bytes a decode step has to read (every weight it
uses once + the cache of the live requests) / its time, against the measured copy bandwidth.
`points`: decode at batch 1 and 64.  A decode step reads > 16 GB of weights, far more than
the 126 MB L2, so no extra flush is made between timed steps (config.l2 says so).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
                max_position_embeddings=40960)


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, 1590.0, 1400.0, "fallback"


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


def model_bytes(cfg, layers):
    h, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qh, kh, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = ((qh + 2 * kh) * d * h + h * qh * d + 3 * F * h + 2 * h + 2 * d) * 2
    return layers * per_layer + V * h * 2 + h * 2, per_layer


def flops_prefill(cfg, layers, T):
    h, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qh, kh, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    mat = (qh + 2 * kh) * d * h + h * qh * d + 3 * F * h
    attn = 2 * 2 * qh * d * T * (T + 1) / 2                  # QK^T and PV over the causal half
    return layers * (2 * T * mat + attn) + 2 * h * V


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--page-size", type=int, default=64, help="tokens per cache page")
    a = ap.parse_args()
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Rust workspace (no Python package, "
                          "no cargo/rustc in this image): pip cannot install it offline"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    if a.warmup < 3:
        a.warmup = 3

    import torch
    from reinfer_b200 import ops
    from reinfer_b200.config import Qwen3Config
    from reinfer_b200.engine import Engine, StepEntry
    from reinfer_b200.engine.llm import LLM
    from reinfer_b200.sampling import SamplingParams

    raw = dict(QWEN3_8B)
    full_layers = raw["num_hidden_layers"]
    layers = a.layers or full_layers
    raw["num_hidden_layers"] = layers
    cfg = Qwen3Config.from_dict(raw)
    hbm_gbs, tf_burst, tf_sust, peak_src = peaks()
    page = a.page_size
    max_b = max(a.batch, 1 if a.no_points else 64)
    ctx_len = a.context
    pool_tokens = max_b * (ctx_len + page) + 4096
    t0 = time.time()
    engine = Engine.from_config(cfg, seed=0, dtype="bfloat16", page_size=page, max_tokens=pool_tokens,
                                max_num_seqs=max_b + 1)
    load_s = time.time() - t0
    gen = torch.Generator().manual_seed(0)
    V = cfg.vocab_size
    kv_bytes_tok = layers * 2 * cfg.num_key_value_heads * cfg.head_dim * 2
    wbytes, _ = model_bytes(raw, layers)

    def ev():
        return torch.cuda.Event(enable_timing=True)

    # ---- prefill: one request of 2,048 tokens ---------------------------------------------
    T = 2048
    pre_ms = []
    for it in range(3):
        toks = torch.randint(0, V, (T,), generator=gen).tolist()
        e0, e1 = ev(), ev()
        torch.cuda.synchronize()
        e0.record()
        engine.step([StepEntry("p", toks, [T - 1])])
        e1.record()
        torch.cuda.synchronize()
        pre_ms.append(e0.elapsed_time(e1))
        engine.finish("p")
    pms = min(pre_ms[1:])
    prefill = {"value": T / pms * 1e3, "tokens": T, "ms": pms,
               "frac": flops_prefill(raw, layers, T) / (pms * 1e-3) / (tf_burst * 1e12), "peak": f"of {peak_src} burst"}

    # ---- decode ---------------------------------------------------------------------------
    def decode_run(B, steps, warmup, through_llm):
        """Fill B requests to ctx_len - steps - warmup tokens, then time `steps` decode steps."""
        # requests admitted first decode a little while the others still run their prompts; leave room
        # so that every request is still alive, and below `context`, when the timed steps end
        start_len = max(ctx_len - steps - warmup - 3 * B - 2, 1)
        llm = LLM(engine=engine, max_batch_tokens=2048, seed=0)
        sp = SamplingParams(temperature=0.0, max_tokens=1 << 20, ignore_eos=True)
        for b in range(B):
            llm.add_request(torch.randint(0, V, (start_len,), generator=gen).tolist(), sp)
        while any(r.in_prefill for r in llm.scheduler.running) or llm.scheduler.waiting:
            llm.step()
        for _ in range(warmup):
            llm.step()
        torch.cuda.synchronize()
        # (1) end to end: K steps through the entry point, wall clock
        w0 = time.perf_counter()
        for _ in range(steps):
            llm.step()
        torch.cuda.synchronize()
        wall = time.perf_counter() - w0
        assert len(llm.scheduler.running) == B and not llm.scheduler.waiting
        kv_tokens = sum(engine.cache.length(r.request_id) for r in llm.scheduler.running)
        # (2) the device alone: the same step's graph and the sampler kernel, K times back to back
        bucket = B if B <= 8 else -(-B // 8) * 8
        graph = max((g for (bk, _w), g in engine._graphs.items() if bk == bucket), key=lambda g: g.meta.numel())
        rows = [r for r in llm.scheduler.running]
        params = [r.params for r in rows]
        rec_args = ([r.seed for r in rows], [len(r.output) for r in rows])
        smp = llm.sampler
        dparams, out_tok = smp.device_records(params, *rec_args), torch.empty(B, dtype=torch.int32, device=engine.device)
        for _ in range(3):
            graph.graph.replay()
            ops.sample(graph.logits, None, dparams, None, smp._work, out_tok, B)
        torch.cuda.synchronize()
        e0, e1 = ev(), ev()
        e0.record()
        for _ in range(steps):
            graph.graph.replay()
            ops.sample(graph.logits, None, dparams, None, smp._work, out_tok, B)
        e1.record()
        torch.cuda.synchronize()
        dev_ms = e0.elapsed_time(e1)
        n_l = (graph.n_launches + 1) * steps            # kernels inside the replayed graph (counted at capture) + sampler
        for r in list(llm.scheduler.running):
            llm.abort(r.request_id)
        return dev_ms / steps, wall / steps * 1e3, n_l, kv_tokens

    clocks = ClockSampler()
    clocks.start()
    ms_dev, ms_wall, n_launch, kv_tokens = decode_run(a.batch, a.steps, a.warmup, True)
    clk = clocks.finish()
    kv_read = kv_tokens * kv_bytes_tok                   # tokens the live requests hold, mid-run
    achieved = (wbytes + kv_read) / (ms_dev * 1e-3) / 1e9
    points = {}
    if not a.no_points:
        for B in (1, 64):
            m, _, _, _ = decode_run(B, max(8, a.steps // 4), 3, True)
            points[f"decode_b{B}"] = B / m * 1e3
    value = a.batch / ms_dev * 1e3
    out = {
        "metric": "decode tok/s (Qwen3-8B shape, bf16, batch %d, context %d)" % (a.batch, ctx_len),
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": ms_dev, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02) drawn on the device, uniform-random token ids",
        "impl": "ours",
        "config": {"model": "Qwen3-8B shape", "layers": layers, "layers_of_model": full_layers,
                   "hidden": cfg.hidden_size, "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": a.batch, "seq_len": ctx_len, "page_size": page, "parallelism": "single GPU",
                   "l2": "inputs (weights+cache per step) larger than L2, no flush", "sampling": "greedy on the GPU"},
        "e2e": {"value": a.batch / ms_wall * 1e3, "unit": "tokens/s", "ms_per_step": ms_wall,
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": a.batch * 4},
        "gpu_launches": n_launch,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
                     "peak_source": f"of {peak_src}"},
        "points": points, "clocks": clk, "load_s": load_s, "kernel_error_word": ops.kernel_error(reset=False),
    }
    # bytes of the int32 block the step uploads (ids, positions, entry, tables: Engine._layout) + sampler records
    B = a.batch
    bucket = B if B <= 8 else -(-B // 8) * 8
    width = 8
    while width < -(-ctx_len // page):
        width *= 2
    from reinfer_b200.engine.engine import Engine as _E
    out["e2e"]["h2d_bytes_per_step"] = 4 * _E._layout(bucket, bucket, bucket, [width])[1] + B * 48
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
