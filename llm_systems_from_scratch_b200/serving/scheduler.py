"""Continuous-batching scheduler (first come, first served) and the request / trace types.

Every engine iteration the scheduler (1) admits waiting requests that have arrived, in arrival
order, as long as the running batch has room, the prefill token budget is not exceeded and the KV
cache can hold the request's whole lifetime (prompt + maximum output, reserved up front so a
running request is never pre-empted), and (2) hands all running requests to one decode step.
Finished requests return their pages immediately, so a request that arrives mid-flight joins the
batch at the next iteration instead of waiting for the batch to drain.

The reference has no serving loop: its ``generate`` (llm-core/llm_core/model.py:187-236) handles one prompt at a
time and ``generate.py`` is a REPL around it.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import numpy as np


@dataclass
class Request:
    rid: int
    prompt: list[int]
    max_new_tokens: int
    arrival: float = 0.0
    eos_token_id: int | None = None
    # runtime state
    pages: list[int] = field(default_factory=list)
    output: list[int] = field(default_factory=list)
    t_first: float | None = None
    t_done: float | None = None
    row: int = -1            # row of the engine's batch arrays while running
    issued: int = 0          # tokens produced on the device so far (the host may not have read the last one yet)

    @property
    def context_len(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def finished(self) -> bool:
        if len(self.output) >= self.max_new_tokens:
            return True
        return bool(self.output) and self.eos_token_id is not None and self.output[-1] == self.eos_token_id


def poisson_trace(num_requests: int, rate: float, prompt_len: tuple[int, int], output_len: tuple[int, int], vocab: int,
                  seed: int = 0) -> list[Request]:
    """Requests with exponential inter-arrival times (``rate`` per second), prompt and output lengths
    uniform in the given inclusive ranges, and uniform random prompt token ids."""
    rng = np.random.default_rng(seed)
    t = np.cumsum(rng.exponential(1.0 / rate, size=num_requests))
    reqs = []
    for i in range(num_requests):
        pl = int(rng.integers(prompt_len[0], prompt_len[1] + 1))
        ol = int(rng.integers(output_len[0], output_len[1] + 1))
        reqs.append(Request(i, rng.integers(0, vocab, size=pl).tolist(), ol, float(t[i])))
    return reqs


class Scheduler:
    def __init__(self, allocator, page_size: int, max_batch: int, max_prefill_tokens: int = 8192,
                 max_context: int = 2560):
        self.alloc = allocator
        self.page_size = page_size
        self.max_batch = max_batch
        self.max_prefill_tokens = max_prefill_tokens
        self.max_context = max_context
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []

    def add(self, req: Request):
        if len(req.prompt) + req.max_new_tokens > self.max_context:
            raise ValueError(f"request {req.rid} needs {len(req.prompt) + req.max_new_tokens} positions, "
                             f"limit is {self.max_context}")
        total = getattr(self.alloc, "num_pages", None)
        if total is not None and self._pages_needed(req) > total:
            # it could never be admitted: refuse it here instead of letting the engine wait for pages forever
            raise ValueError(f"request {req.rid} needs {self._pages_needed(req)} KV pages, the cache has {total}")
        self.waiting.append(req)

    def _pages_needed(self, req: Request) -> int:
        return -(-(len(req.prompt) + req.max_new_tokens) // self.page_size)

    def admit(self, now: float) -> list[Request]:
        """Requests to prefill this iteration (pages already reserved)."""
        batch, tokens = [], 0
        while self.waiting and len(self.running) + len(batch) < self.max_batch:
            req = self.waiting[0]
            if req.arrival > now:
                break
            need = self._pages_needed(req)
            if need > self.alloc.free:
                break                                   # FCFS: do not let later requests overtake
            if batch and tokens + len(req.prompt) > self.max_prefill_tokens:
                break
            self.waiting.popleft()
            req.pages = self.alloc.take(need)
            tokens += len(req.prompt)
            batch.append(req)
        return batch

    def start(self, reqs: list[Request]):
        self.running.extend(reqs)

    def retire(self, now: float) -> list[Request]:
        done = [r for r in self.running if r.finished]
        if done:
            self.running = [r for r in self.running if not r.finished]
            for r in done:
                r.t_done = now
                self.alloc.give(r.pages)
                r.pages = []
        return done

    def finish(self, req: Request):
        """``req`` has produced its last token: return its pages and drop it from the running set."""
        self.running.remove(req)
        self.alloc.give(req.pages)
        req.pages = []

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    def next_arrival(self) -> float | None:
        return self.waiting[0].arrival if self.waiting else None
