"""Observability: per-step console lines in the reference's format, JSONL metrics, CUDA-event
timers, NVTX ranges, GPU statistics and optional wandb.

Reference behaviour kept: one line per step ``[Rank r] Step s: loss = .., lr = .., time = ..s,
tok/s = ..`` (train.py:229), wandb scalars on rank 0 only (train.py:118-119,231-232,260-271) and
``nvidia-smi`` utilisation / memory / temperature (train.py:55-61).  Added: step time measured with
CUDA events (the reference's host timer is unsynchronised in distributed runs), a JSON-lines
file, and serving counters.
"""
from __future__ import annotations

import contextlib
import os
import json
import subprocess
import time

import torch


def get_gpu_stats() -> list[list[str]]:
    """[[utilisation %, memory MiB, temperature C], ...] per GPU, via nvidia-smi; [] if unavailable."""
    try:
        res = subprocess.run(["nvidia-smi", "--query-gpu=utilization.gpu,memory.used,temperature.gpu",
                              "--format=csv,noheader,nounits"], stdout=subprocess.PIPE, timeout=10)
    except (OSError, subprocess.TimeoutExpired):
        return []
    lines = res.stdout.decode("utf-8").strip().split("\n")
    return [ln.split(", ") for ln in lines if ln]


NVTX_ENABLED = os.environ.get("B200_NVTX", "0") == "1"
_NULL = contextlib.nullcontext()


@contextlib.contextmanager
def _nvtx(name: str):
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def nvtx_range(name: str):
    """NVTX range (per block, phase and collective) when ``B200_NVTX=1`` and CUDA is present; otherwise a shared
    no-op context, so the annotations cost nothing in normal runs."""
    if NVTX_ENABLED and torch.cuda.is_available():
        return _nvtx(name)
    return _NULL


class StepTimer:
    """Device-side step time (CUDA events) with a host fallback."""

    def __init__(self, device):
        self.cuda = torch.device(device).type == "cuda"
        self._t0 = None
        self._ev = None

    def start(self):
        if self.cuda:
            self._ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._ev[0].record()
        else:
            self._t0 = time.perf_counter()

    def stop(self) -> float:
        """Seconds since ``start``; synchronises on the end event only."""
        if self.cuda:
            self._ev[1].record()
            self._ev[1].synchronize()
            return self._ev[0].elapsed_time(self._ev[1]) / 1e3
        return time.perf_counter() - self._t0


class MetricsLogger:
    def __init__(self, rank: int = 0, jsonl_path: str | None = None, wandb_run=None):
        self.rank = rank
        self.wandb = wandb_run
        self._f = open(jsonl_path, "a") if (jsonl_path and rank == 0) else None

    def step_line(self, step: int, loss: float, lr: float, step_time: float, tokens_per_sec: float):
        print(f"[Rank {self.rank}] Step {step}: loss = {loss:.4f}, lr = {lr:.6f}, time = {step_time:.4f}s, "
              f"tok/s = {tokens_per_sec:.0f}")

    def log(self, record: dict):
        if self._f is not None:
            self._f.write(json.dumps(record) + "\n")
            self._f.flush()
        if self.wandb is not None:
            self.wandb.log(record)

    def close(self):
        if self._f is not None:
            self._f.close()


class Percentiles:
    """Streaming collection of latencies with percentile queries (serving metrics)."""

    def __init__(self):
        self.values: list[float] = []

    def add(self, v: float):
        self.values.append(v)

    def pct(self, q: float) -> float:
        if not self.values:
            return float("nan")
        s = sorted(self.values)
        k = min(len(s) - 1, max(0, int(round(q / 100.0 * (len(s) - 1)))))
        return s[k]
