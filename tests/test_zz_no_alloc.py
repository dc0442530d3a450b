"""The sampler's entry point that allocates nothing (rb_sample_static), called through its
exported C symbol and compared with the ordinary entry point (rb_sample) on two calls in a
row.  Collected last on purpose: a run that stops at the first failure has by then run every
other test.  It needs nothing from them and passes alone in a fresh process."""
import ctypes
from ctypes import c_int, c_longlong, c_void_p

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _records(rows, temperature, seed, step0):
    from reinfer_b200.sampling.sampler import RECORD
    rec = np.zeros(rows, dtype=RECORD)
    for r in range(rows):
        rec[r] = (temperature, 40 if temperature > 0 else 0, 0.9 if temperature > 0 else 1.0, 0.0, 1.3, 0.0, 0.0, 3,
                  seed + r, step0 + r, 0, 0, 0)                        # (no logit bias)
    return torch.from_numpy(rec.view(np.uint8).copy()).cuda()


def test_static_scratch_sampler_matches_the_ordinary_one():
    from reinfer_b200 import ops
    lib = ops.lib()
    ops.require_device()
    fn = lib.rb_sample_static
    fn.restype = c_int
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    rows, vocab = 5, 30011
    assert rows * vocab <= 2 << 20
    gen = torch.Generator(device="cuda").manual_seed(123)
    for call, temperature in enumerate((0.0, 0.8)):              # two calls in a row, the second over stale scratch
        logits = torch.randn(rows + 2, vocab, device="cuda", generator=gen) * 3
        logits[1, 7] = float("inf")
        row_idx = torch.tensor([6, 0, 1, 3, 2], dtype=torch.int32, device="cuda")
        params = _records(rows, temperature, seed=77 + call, step0=call * 10)
        history = torch.randint(0, vocab, (rows, 64), dtype=torch.int32, device="cuda", generator=gen)
        want = torch.full((rows,), -5, dtype=torch.int32, device="cuda")
        work = torch.empty(rows * vocab, dtype=torch.float32, device="cuda")
        ops.sample(logits, row_idx, params, history, work, want, rows)
        got = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
        rc = fn(c_void_p(logits.data_ptr()), c_longlong(logits.stride(0)), c_void_p(row_idx.data_ptr()),
                c_void_p(params.data_ptr()), c_void_p(history.data_ptr()), c_int(64), c_void_p(got.data_ptr()),
                c_int(rows), c_int(vocab), stream)
        assert rc == 0, lib.rb_last_error().decode()
        torch.cuda.synchronize()
        assert got.tolist() == want.tolist()
        assert all(0 <= t < vocab for t in got.tolist())
    # beyond the built-in array: refused, nothing launched, nothing written
    got.fill_(-7)
    rc = fn(c_void_p(logits.data_ptr()), c_longlong(logits.stride(0)), None, c_void_p(params.data_ptr()), None, c_int(0),
            c_void_p(got.data_ptr()), c_int(rows), c_int((2 << 20) // rows + 1), stream)
    assert rc == -1 and b"built-in array" in lib.rb_last_error()
    torch.cuda.synchronize()
    assert got.tolist() == [-7] * rows
