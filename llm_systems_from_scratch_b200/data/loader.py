"""Random-window batch sampling from a flat token array (np.memmap of uint32).

``sample_batch`` keeps the reference contract (llm-core/llm_core/dataloader.py:8-27): start
offsets are drawn with the global torch RNG from ``[0, len - ctx)``, inputs are ``tokens[i:i+ctx]``
and targets the same window shifted by one, both int64 ``(B, ctx)`` on ``device``.

``BatchSampler`` is the throughput path: windows are gathered by the native loader thread (C++,
``csrc/host_runtime.cpp``) or numpy straight into a reusable pinned staging buffer and copied to the
device on a side stream, one batch ahead of the consumer, so the training stream never waits on the
host.
"""
from __future__ import annotations

import numpy as np
import torch


def sample_batch(tokens, batch_size: int, context_length: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    starts = torch.randint(len(tokens) - context_length, (batch_size,)).numpy()
    window = np.arange(context_length + 1, dtype=np.int64)[None, :] + starts[:, None]
    block = torch.from_numpy(np.asarray(tokens)[window].astype(np.int64))
    x, y = block[:, :-1].contiguous(), block[:, 1:].contiguous()
    if torch.device(device).type == "cuda":
        return x.pin_memory().to(device, non_blocking=True), y.pin_memory().to(device, non_blocking=True)
    return x.to(device), y.to(device)


class BatchSampler:
    """Double-buffered, pinned, prefetching sampler over a token array.

    ``seed`` makes the offset stream reproducible (the reference never seeds); ``rank`` offsets the
    stream so data-parallel ranks draw different windows.
    """

    def __init__(self, tokens, batch_size: int, context_length: int, device, seed: int = 0, rank: int = 0):
        self.tokens = tokens
        self.b, self.ctx = batch_size, context_length
        self.device = torch.device(device)
        self.rng = np.random.default_rng(seed * 1000003 + rank)
        self.cuda = self.device.type == "cuda"
        n = 2 if self.cuda else 1
        self.host = [torch.empty((batch_size, context_length + 1), dtype=torch.int64,
                                 pin_memory=self.cuda) for _ in range(n)]
        self.dev = [torch.empty((batch_size, context_length + 1), dtype=torch.int64, device=self.device)
                    for _ in range(n)] if self.cuda else None
        self.stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self.ready = [None] * n       # H2D copy of slot finished (recorded on the side stream)
        self.consumed = [None] * n    # compute stream finished reading the slot's device buffer
        self.slot = 0
        self._native = None
        try:
            from ..utils import host_runtime
            self._native = host_runtime if host_runtime.available() else None
        except Exception:
            self._native = None
        if self.cuda:
            self._stage(0)

    def _fill(self, buf: torch.Tensor):
        starts = self.rng.integers(0, len(self.tokens) - self.ctx, size=self.b, dtype=np.int64)
        if self._native is not None and isinstance(self.tokens, np.ndarray) and self.tokens.dtype == np.uint32:
            self._native.gather_windows(self.tokens, starts, self.ctx + 1, buf)
            return
        window = np.arange(self.ctx + 1, dtype=np.int64)[None, :] + starts[:, None]
        buf.copy_(torch.from_numpy(np.asarray(self.tokens)[window].astype(np.int64)))

    def _stage(self, slot: int):
        if self.ready[slot] is not None:
            self.ready[slot].synchronize()          # the pinned buffer is no longer being read by a copy
        self._fill(self.host[slot])
        with torch.cuda.stream(self.stream):
            if self.consumed[slot] is not None:
                self.stream.wait_event(self.consumed[slot])
            self.dev[slot].copy_(self.host[slot], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        self.ready[slot] = ev

    def bytes_per_batch(self) -> int:
        """Host-to-device bytes moved per batch."""
        return self.b * (self.ctx + 1) * 8

    def next(self) -> tuple[torch.Tensor, torch.Tensor]:
        """Return (inputs, targets) for this step and start staging the following batch."""
        if not self.cuda:
            self._fill(self.host[0])
            blk = self.host[0]
            return blk[:, :-1].contiguous(), blk[:, 1:].contiguous()
        s = self.slot
        cur = torch.cuda.current_stream()
        cur.wait_event(self.ready[s])
        blk = self.dev[s]
        x, y = blk[:, :-1].contiguous(), blk[:, 1:].contiguous()
        ev = torch.cuda.Event()
        ev.record(cur)
        self.consumed[s] = ev
        self.slot = s ^ 1
        self._stage(self.slot)
        return x, y
