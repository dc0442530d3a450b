"""Trace replay: feed given token ids through the engine step by step and write the
logits at the wanted places.  Nothing is sampled.  This module holds no forward pass,
cache or loader of its own: it builds an `Engine` and calls `Engine.step` /
`Engine.finish`, the ones generation uses.

Input, one JSON object per line on standard input:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, `<out>/<step>.f32` holds the logits
[wanted, vocab] as little-endian float32, in the order of the entries and of `want`.
After every step a line `done <step>` is printed and flushed.
(The reference has no such program; its nearest relatives are the referee's record
format, bench/referee/llama_referee.cpp:17-22, and the scheduler's replay harness,
crates/scheduler/src/replay.rs:180-208.)
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--max-num-seqs", type=int, default=8)
    args = ap.parse_args(argv)

    print("trace_run: loading torch and the kernel library ...", file=sys.stderr, flush=True)
    import numpy as np
    import torch
    from reinfer_b200 import ops
    from reinfer_b200.engine import Engine, StepEntry

    ops.lib()                      # builds at the first call, printing progress lines
    os.makedirs(args.out, exist_ok=True)
    if 64 % args.page_size:
        ap.error("--page-size must divide 64")
    engine = Engine.from_model_dir(args.model, dtype=args.dtype, page_size=args.page_size,
                                   max_tokens=args.max_tokens, max_num_seqs=args.max_num_seqs)
    print(f"trace_run: ready ({engine.cache.total_pages()} pages of {args.page_size} tokens)",
          file=sys.stderr, flush=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in rec.get("entries", [])]
        logits = engine.step(entries)
        if logits is not None and logits.shape[0] > 0:
            arr = logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
            tmp = os.path.join(args.out, f".{step}.f32.tmp")
            arr.tofile(tmp)
            os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        else:
            torch.cuda.synchronize()
        engine.check_status()          # the step is over on the device: a kernel that gave up a wait ends the replay
        for rid in rec.get("end", []):
            engine.finish(rid)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
