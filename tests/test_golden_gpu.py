"""This engine's kernels against numbers that the reference's own kernels produced (tests/golden/
reference_kernels.json, made by tests/golden/make_golden.py from LeonRust/reinfer's unchanged
crates/cuda/kernels): the sampler's draws for given (seed, draw number) - the SplitMix64 stream, the
Gumbel noise and the order of the chain are shared definitions - and the fused per-head norm + rotation."""
import json
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_kernels.json")


@pytest.fixture(scope="module")
def golden():
    with open(PATH) as f:
        return json.load(f)["cases"]


def test_sampler_draws_the_reference_kernels_tokens(golden):
    from reinfer_b200.sampling import Sampler, SamplingParams
    g = golden["gpu_sampler_kernel"]
    logits = torch.tensor([float(v) for v in g["logits"]], dtype=torch.float32, device="cuda").reshape(1, -1)
    s = Sampler(logits.shape[1], 1, "cuda")
    agree = 0
    for c in g["draws"]:
        st = c["settings"]
        window = st.get("window", [])
        p = SamplingParams(temperature=st["temperature"], top_k=st.get("top_k", 0), top_p=st.get("top_p", 1.0),
                           min_p=st.get("min_p", 0.0), repeat_penalty=st.get("rep", 1.0), frequency_penalty=st.get("freq", 0.0),
                           presence_penalty=st.get("pres", 0.0), logit_bias=tuple((int(i), float(v)) for i, v in st.get("bias", [])),
                           repeat_last_n=max(len(window), 1))
        # the reference's draw number is 1-based (its n-th stream output); this engine counts draws from 0
        tok = s.sample(logits, [p], [c["seed"]], [c["draw"] - 1], [window])[0]
        assert c["status"] == 0
        assert tok == c["token"], f"{st} seed {c['seed']} draw {c['draw']}: {tok} for the reference's {c['token']}"
        agree += 1
    assert agree == len(g["draws"]) >= 27


def test_fused_head_norm_and_rotation_match_the_reference_kernels(golden):
    """rb_qknorm_rope_append (per-head RMSNorm, then rotation, in one kernel) on the reference's float16 inputs,
    widened to float32: the reference's float16 results within float16's rounding."""
    from reinfer_b200 import ops
    c = golden["head_norm_then_rope_f16"][0]
    rows, n = c["rows"], c["n"]
    from_bits = lambda b: torch.from_numpy(np.asarray(b, dtype=np.uint16).view(np.float16).astype(np.float32))
    x, w = from_bits(c["x_bits"]).reshape(1, rows * n).cuda(), from_bits(c["w_bits"]).cuda()
    want = from_bits(c["out_bits"]).reshape(rows, n)
    half = n // 2
    inv_freq = (torch.tensor(c["eta"], dtype=torch.float64) ** (-(2.0 * torch.arange(half, dtype=torch.float64)) / n)).float().cuda()
    pos = torch.tensor([c["pos"]], dtype=torch.int32, device="cuda")
    # all rows as query heads, no kv heads, no cache: the kernel's norm + rotation alone
    qkv = x.contiguous()
    q_out = torch.empty(1, rows, n, device="cuda")
    ops.qknorm_rope_append(qkv, w, w, inv_freq, pos, None, q_out, None, rows, 0, n, n, 1, c["eps"])
    got = q_out.reshape(rows, n).cpu()
    assert (got - want).abs().max().item() <= 3e-3 * want.abs().max().item()
