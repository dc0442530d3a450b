"""A few steps of a random-weight model for a profiler to look at:

    python -m reinfer_b200.profile_step --mode decode|prefill --batch B --context N [--layers L] [--steps K]

builds the Qwen3-8B shape (or fewer layers of it), fills B requests to N tokens, runs two
warm-up steps, and brackets K steps of the chosen kind with cudaProfilerStart/Stop, so that
`ncu --profile-from-start off` sees exactly those (the reference brackets its step with event
profilers instead, crates/cuda/src/engine.rs:928-1408).  Decode steps are launched eagerly
(no graph), so every kernel appears as its own launch.
"""
from __future__ import annotations

import argparse
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--mode", choices=["decode", "prefill"], default="decode")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4000)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    a = ap.parse_args(argv)

    import torch
    from . import ops
    from .config import Qwen3Config
    from .engine import Engine, StepEntry

    cfg = Qwen3Config.from_dict(dict(
        architectures=["Qwen3ForCausalLM"], num_hidden_layers=a.layers, hidden_size=4096, num_attention_heads=32,
        num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936, rope_theta=1e6,
        rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960))
    B, N = a.batch, a.context
    eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", page_size=64, max_tokens=B * (N + 64) + 2 * a.prefill_tokens,
                             max_num_seqs=B + 1, cuda_graphs=False)
    g = torch.Generator().manual_seed(0)
    for b in range(B):
        toks = torch.randint(0, cfg.vocab_size, (N,), generator=g).tolist()
        for i in range(0, N, 2048):
            eng.step([StepEntry(b, toks[i:i + 2048], [])])

    def decode():
        return eng.step([StepEntry(b, [5 + b], [0]) for b in range(B)])

    for _ in range(2):
        decode()
    torch.cuda.synchronize()
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


if __name__ == "__main__":
    sys.exit(main())
