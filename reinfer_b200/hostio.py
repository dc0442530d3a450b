"""Small pieces of host <-> device traffic that the engine and the sampler share: a ring of pinned
staging buffers for uploads, and a handle for results that come back one step later."""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch


class PinnedRing:
    """A small ring of pinned int32 buffers; a buffer is reused only after the copy that read
    it has finished (an event per buffer)."""

    def __init__(self, n_buffers: int = 4, capacity: int = 1 << 16):
        self.bufs = [torch.empty(capacity, dtype=torch.int32, pin_memory=True) for _ in range(n_buffers)]
        self.events: List[Optional[torch.cuda.Event]] = [None] * n_buffers
        self.i = 0

    def upload(self, host: np.ndarray, device, into: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Copy the int32 array to the device (into `into`, or a new tensor) on the current stream."""
        n = host.shape[0]
        i = self.i
        self.i = (self.i + 1) % len(self.bufs)
        if self.events[i] is not None:
            self.events[i].synchronize()
        if self.bufs[i].numel() < n:
            self.bufs[i] = torch.empty(max(n, 2 * self.bufs[i].numel()), dtype=torch.int32, pin_memory=True)
        self.bufs[i][:n].numpy()[:] = host
        dev = into if into is not None else torch.empty(n, dtype=torch.int32, device=device)
        dev[:n].copy_(self.bufs[i][:n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[i] = ev
        return dev


class TokenFuture:
    """Token ids on their way from the device to pinned memory; `result()` waits for them."""

    def __init__(self, host: torch.Tensor, rows: int, event: torch.cuda.Event):
        self._host, self._rows, self._event = host, rows, event
        self._done: Optional[List[int]] = None

    def result(self) -> List[int]:
        if self._done is None:
            self._event.synchronize()
            self._done = [int(v) for v in self._host[:self._rows].tolist()]
        return self._done


class TokenDownload:
    """A ring of pinned buffers for the sampled ids of the steps in flight (each step's copy is followed by
    an event; with `depth` buffers a buffer is written again only `depth` steps later)."""

    def __init__(self, max_rows: int, depth: int = 4):
        self.bufs = [torch.empty(max_rows, dtype=torch.int32, pin_memory=True) for _ in range(depth)]
        self.i = 0

    def start(self, device_tokens: torch.Tensor, rows: int) -> TokenFuture:
        buf = self.bufs[self.i]
        self.i = (self.i + 1) % len(self.bufs)
        buf[:rows].copy_(device_tokens[:rows], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return TokenFuture(buf, rows, ev)
