"""Host side of the GPU sampler (csrc/sampler.cu).  The draw of a request at its n-th
generated token is a pure function of (its seed, n, token id): SplitMix64 stream and
Gumbel noise as in the reference (crates/cuda/kernels/sampler_kernel.cu:61-77;
crates/scheduler/src/rng.rs:12-50), so the tokens of a request do not depend on the
batch it was in.

Two ways in.  Serving uses the slots: a request's record (parameters, seed, count of
draws), its ring of recent tokens and the token drawn last are rows of tables on the
device (cache/storage.py), written once when the request is admitted (`assign`); a step
then only launches the kernel (`launch_slots`: no upload, so the launch can be part of a
captured decode graph) and the kernel keeps the rows up to date itself.  `sample` /
`launch` / `fetch` take the records from the host with every call, for callers that
sample logits of their own.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..hostio import PinnedRing, TokenDownload, TokenFuture
from .params import SamplingParams

HIST_CAP = 64
_MASK64 = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15

RECORD = np.dtype([("temperature", "<f4"), ("top_k", "<i4"), ("top_p", "<f4"), ("min_p", "<f4"),
                   ("repeat_penalty", "<f4"), ("frequency_penalty", "<f4"), ("presence_penalty", "<f4"),
                   ("hist_len", "<i4"), ("seed", "<u8"), ("step", "<u8"), ("bias", "<u8"), ("bias_len", "<i4"),
                   ("hist_window", "<i4")])
BIAS_CAP = 1024                     # logit_bias entries a request may bring


def _mix(z: int) -> int:
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    return z ^ (z >> 31)


def splitmix64(x: int) -> int:
    """mix(x + golden)  (crates/scheduler/src/rng.rs:24-30)."""
    return _mix((x + GOLDEN) & _MASK64)


def request_seed(base_seed: int, arrival: int) -> int:
    """Seed of a request that brought none: splitmix64(base ^ arrival number)
    (bin/reinfer/src/sched_loop.rs:650-653)."""
    return splitmix64((base_seed ^ arrival) & _MASK64)


def history_ring(drawn: Sequence[int], window: int):
    """(ring, valid entries) of a request that has drawn the tokens `drawn`: the penalties look at the last
    `window` tokens the request has SAMPLED, never at its prompt (crates/cuda/src/sampler.rs:109-111 and :369:
    the history is fed by `history.push(token)` after each draw), and the n-th draw lives at ring index
    n mod window, where the kernel puts the draws that follow.  A preempted request keeps its output, so its
    ring is the same when it returns."""
    ring = np.zeros(max(window, 0), dtype=np.int32)
    n = len(drawn)
    for j in range(max(0, n - window), n):
        ring[j % window] = drawn[j]
    return ring, min(n, max(window, 0))


class Sampler:
    def __init__(self, vocab_size: int, max_rows: int, device, storage=None):
        """storage: the engine's CacheStorage, whose slot rows the slot-driven way works on (None: only the
        host-driven way is used)."""
        self.vocab = int(vocab_size)
        self.device = torch.device(device)
        self.max_rows = int(max_rows)
        if ops.sample_params_size() != RECORD.itemsize:
            raise ops.KernelError("the sampler's record layout differs between library and Python")
        self._work = torch.empty((self.max_rows, self.vocab), dtype=torch.float32, device=self.device)
        self.storage = storage
        if storage is not None:
            if storage.slot_records.shape[1] != RECORD.itemsize:
                raise ops.KernelError("the slots' record rows have another size than the sampler's record")
            self._ring = PinnedRing(n_buffers=8, capacity=256)
            self._download = TokenDownload(self.max_rows)
            self.out_tokens = torch.zeros(self.max_rows, dtype=torch.int32, device=self.device)
            self._slot_bias = None                  # [slots, BIAS_CAP, 2] int32, made when a request first brings a bias
        self._host_params = torch.empty(self.max_rows * RECORD.itemsize, dtype=torch.uint8, pin_memory=True)
        self._host_hist = torch.empty((self.max_rows, HIST_CAP), dtype=torch.int32, pin_memory=True)
        self._host_out = torch.empty(self.max_rows, dtype=torch.int32, pin_memory=True)
        self._host_bias = self._dev_bias = None      # [rows, BIAS_CAP, 2] int32 (id, float bits): made when first needed
        self._done = torch.cuda.Event()

    # ---- the slot-driven way ---------------------------------------------------------------------
    def assign(self, slot: int, params: SamplingParams, seed: int, drawn: Sequence[int]) -> None:
        """A request moves into `slot` (admitted, or back after a preemption) having drawn the tokens `drawn` so
        far: write its record, and its ring of recent tokens if a penalty is on.  The n-th draw lives at ring
        index n mod window, so the kernel goes on where the host left off."""
        st = self.storage
        pen = params.repeat_penalty > 1.0 or params.frequency_penalty != 0.0 or params.presence_penalty != 0.0
        window = min(int(params.repeat_last_n), st.slot_history.shape[1]) if pen else 0
        n = len(drawn)
        ring, valid = history_ring(drawn, window)
        rec = np.zeros(1, dtype=RECORD)
        rec[0] = (params.temperature, params.top_k, params.top_p, params.min_p, params.repeat_penalty,
                  params.frequency_penalty, params.presence_penalty, valid, seed & _MASK64, n, 0, 0, window)
        if params.logit_bias:
            if self._slot_bias is None:
                self._slot_bias = torch.zeros((st.slot_records.shape[0], BIAS_CAP, 2), dtype=torch.int32, device=self.device)
            pairs = np.zeros((len(params.logit_bias), 2), dtype=np.int32)
            pairs[:, 0] = [int(i) for i, _ in params.logit_bias]
            pairs[:, 1] = np.asarray([float(v) for _, v in params.logit_bias], dtype=np.float32).view(np.int32)
            self._ring.upload(pairs.reshape(-1), self.device, into=self._slot_bias[slot].view(-1))
            rec[0]["bias"] = self._slot_bias.data_ptr() + slot * BIAS_CAP * 8
            rec[0]["bias_len"] = len(params.logit_bias)
        self._ring.upload(rec.view(np.int32), self.device, into=st.slot_records[slot].view(torch.int32))
        if valid:
            self._ring.upload(ring, self.device, into=st.slot_history[slot])

    def launch_slots(self, logits: torch.Tensor, row_slot: torch.Tensor, rows: int) -> None:
        """One token for each of the first `rows` rows of `logits`, row r for the request in slot row_slot[r]; the
        tokens go to the slots and to `out_tokens`.  Nothing but the launch happens here."""
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows exceed the sampler's {self.max_rows}")
        st = self.storage
        ops.sample_slots(logits, row_slot, st.slot_records.view(-1), st.slot_history, st.slot_token, self._work,
                         self.out_tokens, rows)

    def download(self, rows: int) -> TokenFuture:
        """Start the copy of the last launch's tokens to pinned memory; the result is read when it is needed."""
        return self._download.start(self.out_tokens, rows)

    # ---- the host-driven way -----------------------------------------------------------------------
    def device_records(self, params: Sequence[SamplingParams], seeds: Sequence[int], steps: Sequence[int]) -> torch.Tensor:
        """The kernel's per-row records for rows without penalties, on the device (for callers that
        launch `ops.sample` themselves)."""
        rec = np.zeros(len(params), dtype=RECORD)
        for r, p in enumerate(params):
            rec[r] = (p.temperature, p.top_k, p.top_p, p.min_p, 1.0, 0.0, 0.0, 0, seeds[r] & _MASK64, steps[r], 0, 0, 0)
        return torch.from_numpy(rec.view(np.uint8).copy()).to(self.device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               steps: Sequence[int], histories: Optional[Sequence[Sequence[int]]] = None) -> List[int]:
        """One token per row of `logits` ([rows, vocab] float32 on the device).  Returns host ints
        (-1 for a row without a finite logit).  Blocks until the tokens are on the host."""
        return self.fetch(self.launch(logits, params, seeds, steps, histories))

    def fetch(self, rows: int) -> List[int]:
        """The tokens of the last `launch` (waits for them)."""
        if rows == 0:
            return []
        self._done.synchronize()
        return [int(v) for v in self._host_out[:rows].tolist()]

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               steps: Sequence[int], histories: Optional[Sequence[Sequence[int]]] = None) -> int:
        """Launch the sampler and the copy of its tokens to pinned memory; returns the row count for `fetch`."""
        rows = logits.shape[0]
        if rows == 0:
            return 0
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows exceed the sampler's {self.max_rows}")
        rec = np.zeros(rows, dtype=RECORD)
        hist = self._host_hist.numpy()
        any_hist = False
        first = params[0]
        if all(p is first for p in params):                      # the common case: one parameter set for the batch
            rec["temperature"], rec["top_k"], rec["top_p"], rec["min_p"] = first.temperature, first.top_k, first.top_p, first.min_p
            rec["repeat_penalty"], rec["frequency_penalty"] = first.repeat_penalty, first.frequency_penalty
            rec["presence_penalty"] = first.presence_penalty
        else:
            for r, p in enumerate(params):
                rec[r] = (p.temperature, p.top_k, p.top_p, p.min_p, p.repeat_penalty, p.frequency_penalty,
                          p.presence_penalty, 0, 0, 0, 0, 0, 0)
        rec["seed"] = np.fromiter((sd & _MASK64 for sd in seeds), dtype=np.uint64, count=rows)
        rec["step"] = np.fromiter(steps, dtype=np.uint64, count=rows)
        for r, p in enumerate(params):
            pen = p.repeat_penalty > 1.0 or p.frequency_penalty != 0.0 or p.presence_penalty != 0.0
            if pen and histories is not None and p.repeat_last_n > 0:
                h = histories[r](p.repeat_last_n) if callable(histories[r]) else list(histories[r])[-p.repeat_last_n:]
                hist[r, :len(h)] = h
                rec[r]["hist_len"] = len(h)
                any_hist = any_hist or bool(h)
        if any(p.logit_bias for p in params):
            # logit_bias (sampler_kernel.cu:161-163,198-205): the pairs go up beside the records, which point at them
            if self._dev_bias is None:
                self._host_bias = torch.zeros((self.max_rows, BIAS_CAP, 2), dtype=torch.int32, pin_memory=True)
                self._dev_bias = torch.zeros((self.max_rows, BIAS_CAP, 2), dtype=torch.int32, device=self.device)
            hb = self._host_bias.numpy()
            for r, p in enumerate(params):
                n = len(p.logit_bias)
                if n:
                    hb[r, :n, 0] = np.fromiter((int(i) for i, _ in p.logit_bias), dtype=np.int32, count=n)
                    hb[r, :n, 1] = np.fromiter((float(v) for _, v in p.logit_bias), dtype=np.float32, count=n).view(np.int32)
                    rec[r]["bias"] = self._dev_bias.data_ptr() + r * BIAS_CAP * 8
                    rec[r]["bias_len"] = n
            self._dev_bias[:rows].copy_(self._host_bias[:rows], non_blocking=True)
        self._host_params.numpy()[:rows * RECORD.itemsize] = rec.view(np.uint8)
        dparams = self._host_params[:rows * RECORD.itemsize].to(self.device, non_blocking=True)
        dhist = self._host_hist[:rows].to(self.device, non_blocking=True) if any_hist else None
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        ops.sample(logits, None, dparams, dhist, self._work, out, rows)
        self._host_out[:rows].copy_(out, non_blocking=True)
        self._done.record()
        return rows
