"""Command line in the reference's manner: `reinfer run <model> [-n MAX_TOKENS] [-t TEMP]
[--top-k K] [--top-p P] [--repeat-penalty R] [--seed S] [--max-model-len N] [--perf]
[prompt ...]` (bin/reinfer/src/main.rs:246-294; defaults: -n 256, -t 1.0).  The engine
works on token ids, so the prompt is a list of integers (separated by blanks or commas),
from the arguments or, when there are none, from standard input; the generated ids are
printed on one line.  `--perf` adds the reference's machine-readable line
(main.rs:700-727).  The model is a local folder, or a name looked up under `$REINFER_MODEL_DIR`
(default `~/.reinfer/models`; main.rs:540-558 - nothing is ever downloaded here).  `--backend`
takes the reference's names; only `auto` and `cuda` run (main.rs:483-509).  `reinfer random-model`
writes a model folder with seeded random weights.  `reinfer bench --shape qwen3-8b|4b|32b|<config.json>
--batch 1,8,64 --prompt-len 2048 --decode-len N` measures a random-weight model of that shape (the
reference measures through `run --perf` and its server's load generator, main.rs:700-727).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def _ids(words):
    out = []
    for w in words:
        for part in w.replace(",", " ").split():
            out.append(int(part))
    return out


def resolve_model_dir(model: str) -> str:
    """A local path wins; else `<model root>/<model>` if a config.json lies there."""
    if os.path.isdir(model) or os.path.isfile(os.path.join(model, "config.json")):
        return model
    root = os.path.expanduser(os.environ.get("REINFER_MODEL_DIR") or os.path.join("~", ".reinfer", "models"))
    found = os.path.join(root, model)
    if os.path.isfile(os.path.join(found, "config.json")):
        return found
    raise FileNotFoundError(f"model not found locally: {model!r} (tried {found!r}); give a folder with config.json "
                            f"and safetensors, or set REINFER_MODEL_DIR")


def cmd_run(a) -> int:
    if a.backend not in ("auto", "cuda"):
        print(f"error: backend {a.backend!r} is not built here; this engine runs on cuda (B200) only", file=sys.stderr)
        return 2
    try:
        a.model = resolve_model_dir(a.model)
    except FileNotFoundError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    from .engine.llm import LLM
    from .sampling.params import SamplingParams
    prompt = _ids(a.prompt) if a.prompt else _ids(sys.stdin.read().split())
    if not prompt:
        print("error: empty prompt (give token ids as arguments or on standard input)", file=sys.stderr)
        return 2
    t0 = time.perf_counter()
    llm = LLM(a.model, dtype=a.dtype, max_model_len=a.max_model_len, page_size=a.page_size,
              num_pages=a.num_pages, max_num_seqs=a.max_num_seqs, max_batch_tokens=a.max_batch_tokens,
              seed=a.seed or 0, admission=a.admission)
    load_s = time.perf_counter() - t0
    sp = SamplingParams(temperature=a.temperature, top_k=a.top_k or 0, top_p=a.top_p if a.top_p is not None else 1.0,
                        min_p=a.min_p or 0.0, repeat_penalty=a.repeat_penalty or 1.0, seed=a.seed,
                        max_tokens=a.max_tokens)
    t1 = time.perf_counter()
    rid = llm.add_request(prompt, sp)
    first = None
    while llm.has_work():
        llm.step()
        if first is None and llm.requests[rid].output:
            first = time.perf_counter() - t1
    dt = time.perf_counter() - t1
    r = llm.requests[rid]
    print(" ".join(str(t) for t in r.output))
    n = len(r.output)
    tpot = (dt - (first or 0.0)) / max(n - 1, 1) * 1e3
    print(f"{n} tokens in {dt:.3f}s (≈{n / dt if dt > 0 else 0:.1f} tok/s, first-token {(first or 0) * 1e3:.1f} ms), "
          f"finish={r.finish_reason}", file=sys.stderr)
    for line in llm.profile_report():
        print(line, file=sys.stderr)
    if a.perf:
        print(f"PERF model={a.model} dtype={a.dtype} load_s={load_s:.2f} prompt_tokens={len(prompt)} "
              f"new_tokens={n} ttft_ms={(first or 0) * 1e3:.3f} tpot_ms={tpot:.3f} "
              f"tok_s={(n - 1) / (dt - (first or 0)) if n > 1 and dt > (first or 0) else 0:.2f} "
              f"preemptions={llm.scheduler.stats['preemptions']}")
    return 0


def cmd_random_model(a) -> int:
    import torch
    from .config.registry import resolve_architecture
    from .weights.loader import write_random_model
    with open(a.config) as f:
        raw = json.load(f)
    arch = resolve_architecture(raw)
    cfg = arch.config_cls.from_dict(raw)
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[a.dtype]
    print(write_random_model(a.out, cfg, a.seed, dt))
    return 0


def cmd_bench(a) -> int:
    """Prefill and decode throughput of a random-weight model of a given shape (reinfer_b200/measure.py)."""
    from . import measure
    batches = [int(b) for b in a.batch.split(",") if b]
    context = a.context or a.prompt_len + a.decode_len
    page = a.page_size
    need = max(batches) * (context + page) + 2 * a.prompt_len + 4096
    hbm, tf, _, src = measure.peaks()
    b = measure.Bench(a.shape, layers=a.layers, page_size=page, dtype=a.dtype, pool_tokens=need,
                      max_num_seqs=max(batches) + 1, seed=a.seed)
    print(f"{os.path.basename(measure.shape_path(a.shape))}: {b.layers} of {b.full_layers} layers, {b.weight_bytes / 1e9:.2f} GB "
          f"of weights a step, {b.kv_bytes_per_token} B of cache a token, pages of {page}; peaks {src}: {hbm:.0f} GB/s, "
          f"{tf:.0f} TFLOP/s", file=sys.stderr)
    out = {"shape": a.shape, "layers": b.layers, "dtype": a.dtype, "page_size": page}
    p = b.prefill(a.prompt_len)
    out["prefill"] = {"tokens": a.prompt_len, "ms": p["ms"], "tokens_per_s": p["value"],
                      "frac_of_peak": p["flops"] / (p["ms"] * 1e-3) / (tf * 1e12)}
    print(f"prefill {a.prompt_len:6d} tokens: {p['ms']:8.2f} ms  {p['value']:10.0f} tok/s  {100 * out['prefill']['frac_of_peak']:5.1f} % of the "
          f"tensor-core peak", file=sys.stderr)
    out["decode"] = []
    for B in batches:
        r = b.decode(B, a.decode_len, 3, context)
        frac = r["bytes"] / (r["ms_device"] * 1e-3) / 1e9 / hbm
        out["decode"].append({"batch": B, "context": context, "ms_device": r["ms_device"], "ms_e2e": r["ms_e2e"],
                              "tokens_per_s": B / r["ms_device"] * 1e3, "e2e_tokens_per_s": B / r["ms_e2e"] * 1e3,
                              "frac_of_bandwidth": frac})
        print(f"decode  batch {B:4d} at {context:6d}: {r['ms_device']:8.3f} ms/step  {B / r['ms_device'] * 1e3:10.1f} tok/s on the device, "
              f"{B / r['ms_e2e'] * 1e3:10.1f} end to end  {100 * frac:5.1f} % of the copy bandwidth", file=sys.stderr)
    if a.segments:
        for kind in ("decode", "prefill"):
            seg = b.segments(kind, B=batches[0], context=context, T=a.prompt_len)
            print(f"-- one eager {kind} step by segment --", file=sys.stderr)
            print("\n".join(measure.segment_table(seg, hbm, tf)), file=sys.stderr)
    print(json.dumps(out))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="reinfer", description="B200-native inference engine (token ids in, token ids out)")
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("run", help="generate from a prompt of token ids")
    r.add_argument("model", help="local model folder (config.json + safetensors), or a name under $REINFER_MODEL_DIR")
    r.add_argument("--backend", choices=["auto", "cuda", "ascend", "cpu"], default="auto")
    r.add_argument("-n", dest="max_tokens", type=int, default=256, metavar="MAX_TOKENS", help="max new tokens")
    r.add_argument("-t", dest="temperature", type=float, default=1.0, metavar="TEMP", help="0 = greedy")
    r.add_argument("--top-k", type=int, default=None, metavar="K")
    r.add_argument("--top-p", type=float, default=None, metavar="P")
    r.add_argument("--min-p", type=float, default=None, metavar="P")
    r.add_argument("--repeat-penalty", type=float, default=None, metavar="PENALTY")
    r.add_argument("--seed", type=int, default=None, metavar="SEED")
    r.add_argument("--max-model-len", type=int, default=None, metavar="N")
    r.add_argument("--perf", action="store_true", help="print a machine-parseable PERF line")
    r.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    r.add_argument("--page-size", type=int, default=64)
    r.add_argument("--num-pages", type=int, default=None)
    r.add_argument("--max-num-seqs", type=int, default=8)
    r.add_argument("--max-batch-tokens", type=int, default=2048)
    r.add_argument("--admission", choices=["pages", "estimate"], default="pages",
                   help="estimate: also ask that the estimated peak of the running requests fits the cache")
    r.add_argument("prompt", nargs="*", help="token ids; standard input when absent")
    r.set_defaults(fn=cmd_run)
    m = sub.add_parser("random-model", help="write a model folder with seeded random weights")
    m.add_argument("--config", required=True, help="a config.json of a registered architecture")
    m.add_argument("--out", required=True)
    m.add_argument("--seed", type=int, default=0)
    m.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    m.set_defaults(fn=cmd_random_model)
    b = sub.add_parser("bench", help="throughput of a random-weight model of a given shape")
    b.add_argument("--shape", default="qwen3-8b", help="qwen3-8b, qwen3-4b, qwen3-32b (or 8b, 4b, 32b), or a config.json")
    b.add_argument("--batch", default="1,8,64", help="decode batch sizes, comma separated")
    b.add_argument("--prompt-len", type=int, default=2048)
    b.add_argument("--decode-len", type=int, default=32, help="timed decode steps per batch size")
    b.add_argument("--context", type=int, default=None, help="tokens a request holds at the end (default prompt + decode)")
    b.add_argument("--dtype", choices=["bfloat16"], default="bfloat16")
    b.add_argument("--page-size", type=int, default=16)
    b.add_argument("--layers", type=int, default=None, help="build only this many layers of the shape")
    b.add_argument("--seed", type=int, default=0)
    b.add_argument("--segments", action="store_true", help="also time one eager step of each kind launch by launch")
    b.set_defaults(fn=cmd_bench)
    a, extra = ap.parse_known_args(argv)
    if extra:
        # token ids that follow options (argparse binds a '*' positional before it sees them)
        if a.cmd != "run" or not all(e.replace(",", "").lstrip("-").isdigit() for e in extra):
            ap.error("unrecognized arguments: " + " ".join(extra))
        a.prompt = list(a.prompt) + extra
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
