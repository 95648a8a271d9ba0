"""Online serving: the continuous-batching engine on a thread of its own, fed by a thread-safe queue, and an HTTP
front end for it.

``EngineServer`` owns the engine loop.  Callers (any thread, any asyncio loop) ``submit`` token ids and get a
``concurrent.futures.Future`` that resolves with a ``Completion`` (the generated ids, time to first token, total
latency).  The loop is the one ``ServingEngine.run`` uses for a recorded trace - admit, prefill, one decode step,
collect - except that arrivals come from the queue as they happen: a request that arrives while others are decoding
joins the batch at the next iteration.  The engine itself is only ever touched by the loop thread.

``build_app`` wraps a server in a small FastAPI application (``POST /generate``, ``GET /health``, ``GET /stats``);
``serve.py --http PORT`` runs it under uvicorn.  The reference has no serving loop (its ``generate`` handles one
prompt at a time, llm-core/llm_core/model.py:187-236, behind the REPL of generate.py).
"""
from __future__ import annotations

import itertools
import queue
import threading
import time
from concurrent.futures import Future
from dataclasses import dataclass

from .scheduler import Request

try:        # the HTTP front end is optional; the engine server itself needs none of this
    from pydantic import BaseModel

    class GenerateRequest(BaseModel):
        prompt: str | None = None
        prompt_ids: list[int] | None = None
        max_new_tokens: int | None = None
        eos_token_id: int | None = None
        stream: bool = False
except ImportError:      # pragma: no cover
    GenerateRequest = None


@dataclass
class Completion:
    request_id: int
    output_ids: list[int]
    ttft_s: float | None        # arrival -> first token on the host
    latency_s: float | None     # arrival -> last token on the host
    cancelled: bool = False     # stopped by ``cancel`` before it had all its tokens


class QueueFull(RuntimeError):
    """More requests are waiting than the server was told to hold; the caller should retry later."""


class EngineServer:
    def __init__(self, engine, idle_wait_s: float = 0.002, max_waiting: int | None = None):
        self.engine = engine
        self.idle_wait_s = idle_wait_s
        self.max_waiting = max_waiting       # back-pressure: submissions beyond this many waiting requests are refused
        self._inbox: queue.Queue = queue.Queue()
        self._ids = itertools.count()
        self._id_lock = threading.Lock()
        self._live: dict[int, tuple[Request, Future]] = {}
        self._streams: dict[int, list] = {}        # request id -> [callback, tokens already delivered]
        self._cancelled: set[int] = set()
        self.ttft_s: list[float] = []              # of completed requests (bounded: the newest 4096)
        self.latency_s: list[float] = []
        self.output_tokens = 0
        self._stop = threading.Event()
        self._error: BaseException | None = None
        self._thread: threading.Thread | None = None
        self.completed = 0

    # ------------------------------------------------------------------ client side (any thread)
    def submit(self, prompt_ids: list[int], max_new_tokens: int, eos_token_id: int | None = None,
               on_tokens=None) -> Future:
        """Queue one request; the future resolves with a ``Completion`` or raises what the engine raised for it
        (a prompt longer than the context, a request that can never fit in the KV cache).  ``on_tokens(ids)`` is called
        on the loop thread with every batch of new token ids as they reach the host (streaming); keep it short."""
        if self._error is not None:
            raise RuntimeError("the engine loop has stopped") from self._error
        if not prompt_ids or max_new_tokens < 1:
            raise ValueError("a request needs at least one prompt token and one token to generate")
        if self.max_waiting is not None and len(self.engine.sched.waiting) + self._inbox.qsize() >= self.max_waiting:
            raise QueueFull(f"{self.max_waiting} requests are already waiting")
        fut: Future = Future()
        with self._id_lock:
            fut.request_id = next(self._ids)         # what ``cancel`` takes
        self._inbox.put(("add", fut.request_id, list(map(int, prompt_ids)), int(max_new_tokens), eos_token_id, fut,
                         on_tokens))
        return fut

    def cancel(self, request_id: int) -> None:
        """Ask the loop to stop a request (a client that went away): its future resolves with what it has so far and
        ``cancelled=True``; its row and KV pages are free for the next request at once.  Unknown or finished ids are
        ignored."""
        self._inbox.put(("cancel", request_id))

    def generate(self, prompt_ids: list[int], max_new_tokens: int, eos_token_id: int | None = None,
                 timeout: float | None = None) -> Completion:
        return self.submit(prompt_ids, max_new_tokens, eos_token_id).result(timeout)

    def stats(self) -> dict:
        eng = self.engine
        return {"running": len(eng.sched.running), "waiting": len(eng.sched.waiting) + self._inbox.qsize(),
                "completed": self.completed, "output_tokens": self.output_tokens,
                "kv_pages": eng.cache.num_pages, "kv_occupancy": eng.cache.occupancy(),
                "prefill_tokens": eng.stats["prefill_tokens"], "decode_steps": eng.stats["decode_steps"],
                "alive": self._thread is not None and self._thread.is_alive() and self._error is None}

    # ------------------------------------------------------------------ loop thread
    def start(self, warmup: bool = True):
        if self._thread is None:
            eng = self.engine
            eng._realtime, eng._virtual = True, float("inf")
            eng._t0 = time.perf_counter()
            if warmup:
                eng.warmup()             # decode graphs are captured before the first request, not during it
            elif not hasattr(eng, "_row_req"):
                eng._rows_init()
            self._thread = threading.Thread(target=self._loop, daemon=True, name="engine-loop")
            self._thread.start()
        return self

    def stop(self, timeout: float = 10.0):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout)
        for _, fut in list(self._live.values()):
            if not fut.done():
                fut.set_exception(RuntimeError("server stopped before the request finished"))
        self._live.clear()

    def _take(self, block_s: float):
        """Move queued submissions into the scheduler; blocks up to ``block_s`` when there is nothing else to do."""
        eng = self.engine
        try:
            item = self._inbox.get(timeout=block_s) if block_s > 0 else self._inbox.get_nowait()
        except queue.Empty:
            return
        while True:
            if item[0] == "cancel":
                live = self._live.get(item[1])
                if live is not None and eng.cancel(live[0]):
                    self._cancelled.add(item[1])
            else:
                _, rid, prompt, max_new, eos, fut, on_tokens = item
                req = Request(rid, prompt, max_new, arrival=eng._clock(), eos_token_id=eos)
                try:
                    eng.sched.add(req)       # validates against the context length and the cache capacity
                    self._live[req.rid] = (req, fut)
                    if on_tokens is not None:
                        self._streams[req.rid] = [on_tokens, 0]
                except Exception as e:       # noqa: BLE001 - the caller gets the scheduler's verdict
                    fut.set_exception(e)
            try:
                item = self._inbox.get_nowait()
            except queue.Empty:
                return

    def _loop(self):
        eng = self.engine
        try:
            if eng.cuda:                     # the current device is per thread and starts at 0 in a new one
                import torch
                torch.cuda.set_device(eng.device)
            while not self._stop.is_set():
                busy = bool(eng.sched.running or eng.sched.waiting or eng._pending)
                self._take(0.0 if busy else self.idle_wait_s)
                if eng.sched.running or eng.sched.waiting or eng._pending:
                    eng.step(eng._clock())
                elif not self._cancelled:
                    continue
                for rid, st in list(self._streams.items()):          # streaming: hand over what is new
                    r = self._live[rid][0]
                    if len(r.output) > st[1]:
                        new, st[1] = r.output[st[1]:], len(r.output)
                        try:
                            st[0](list(new))
                        except Exception:        # noqa: BLE001 - a client's callback must not stop the loop
                            self._streams.pop(rid, None)
                for rid in [rid for rid, (r, _) in self._live.items() if r.t_done is not None]:
                    r, fut = self._live.pop(rid)
                    self._streams.pop(rid, None)
                    self.completed += 1
                    self.output_tokens += len(r.output)
                    ttft = None if r.t_first is None else r.t_first - r.arrival
                    if ttft is not None:
                        self.ttft_s.append(ttft)
                    self.latency_s.append(r.t_done - r.arrival)
                    del self.ttft_s[:-4096], self.latency_s[:-4096]
                    was_cancelled = rid in self._cancelled
                    self._cancelled.discard(rid)
                    fut.set_result(Completion(rid, list(r.output), ttft, r.t_done - r.arrival, was_cancelled))
        except BaseException as e:           # noqa: BLE001 - surfaces in every pending and future request
            self._error = e
            for _, fut in list(self._live.values()):
                if not fut.done():
                    fut.set_exception(e)
            self._live.clear()
            self._streams.clear()


def build_app(server: EngineServer, tokenizer=None, default_max_new_tokens: int = 128):
    """FastAPI application around a started ``EngineServer``.

    ``POST /generate`` takes ``{"prompt_ids": [...]}`` or, with a tokenizer, ``{"prompt": "text"}``, plus optional
    ``max_new_tokens``, ``eos_token_id`` and ``stream``; it answers with the generated ids (and text), the time to
    first token and the latency in milliseconds - or, with ``"stream": true``, with server-sent events, one
    ``data: {"output_ids": [...]}`` per batch of new tokens and a final event that carries the timings.
    ``GET /metrics`` is a Prometheus text exposition of the server's counters.  Requests are served concurrently by
    the one engine loop."""
    import asyncio
    import json

    from fastapi import FastAPI, HTTPException
    from fastapi.responses import PlainTextResponse, StreamingResponse

    app = FastAPI(title="B200 LLM serving")

    @app.get("/health")
    def health():
        s = server.stats()
        if not s["alive"]:
            raise HTTPException(status_code=503, detail="engine loop is not running")
        return {"status": "ok"}

    @app.get("/stats")
    def stats():
        return server.stats()

    @app.get("/metrics")
    def metrics():
        s = server.stats()
        pct = lambda xs, q: sorted(xs)[min(len(xs) - 1, int(q * len(xs)))] if xs else float("nan")
        lines = ["# TYPE llm_requests_completed_total counter", f"llm_requests_completed_total {s['completed']}",
                 "# TYPE llm_output_tokens_total counter", f"llm_output_tokens_total {s['output_tokens']}",
                 "# TYPE llm_prefill_tokens_total counter", f"llm_prefill_tokens_total {s['prefill_tokens']}",
                 "# TYPE llm_decode_steps_total counter", f"llm_decode_steps_total {s['decode_steps']}",
                 "# TYPE llm_requests_running gauge", f"llm_requests_running {s['running']}",
                 "# TYPE llm_requests_waiting gauge", f"llm_requests_waiting {s['waiting']}",
                 "# TYPE llm_kv_cache_occupancy gauge", f"llm_kv_cache_occupancy {s['kv_occupancy']}",
                 "# TYPE llm_ttft_seconds summary",
                 f'llm_ttft_seconds{{quantile="0.5"}} {pct(server.ttft_s, 0.5)}',
                 f'llm_ttft_seconds{{quantile="0.99"}} {pct(server.ttft_s, 0.99)}',
                 "# TYPE llm_request_latency_seconds summary",
                 f'llm_request_latency_seconds{{quantile="0.5"}} {pct(server.latency_s, 0.5)}',
                 f'llm_request_latency_seconds{{quantile="0.99"}} {pct(server.latency_s, 0.99)}']
        return PlainTextResponse("\n".join(lines) + "\n")

    @app.post("/generate")
    async def generate(body: GenerateRequest):
        if body.prompt_ids is not None:
            ids = body.prompt_ids
        elif body.prompt is not None and tokenizer is not None:
            ids = tokenizer.encode(body.prompt)
        else:
            raise HTTPException(status_code=422, detail="give prompt_ids, or prompt when the server has a tokenizer")
        n_new = body.max_new_tokens or default_max_new_tokens
        if body.stream:
            loop = asyncio.get_running_loop()
            chunks: asyncio.Queue = asyncio.Queue()
            try:
                fut = server.submit(ids, n_new, body.eos_token_id,
                                    on_tokens=lambda new: loop.call_soon_threadsafe(chunks.put_nowait, new))
            except QueueFull as e:
                raise HTTPException(status_code=503, detail=str(e), headers={"Retry-After": "1"})
            except (ValueError, RuntimeError) as e:
                raise HTTPException(status_code=400, detail=str(e))
            done_fut = asyncio.wrap_future(fut)

            async def events():
                try:
                    async for chunk in _events():
                        yield chunk
                finally:
                    if not done_fut.done():          # the client went away: free the request's row and pages now
                        server.cancel(fut.request_id)

            async def _events():
                while True:
                    getter = asyncio.ensure_future(chunks.get())
                    finished, _ = await asyncio.wait({getter, done_fut}, return_when=asyncio.FIRST_COMPLETED)
                    if getter in finished:
                        yield "data: " + json.dumps({"output_ids": getter.result()}) + "\n\n"
                        continue
                    getter.cancel()
                    while not chunks.empty():      # what arrived together with the completion
                        yield "data: " + json.dumps({"output_ids": chunks.get_nowait()}) + "\n\n"
                    if done_fut.exception() is not None:
                        yield "data: " + json.dumps({"error": str(done_fut.exception())}) + "\n\n"
                    else:
                        d = done_fut.result()
                        yield "data: " + json.dumps({"done": True, "request_id": d.request_id,
                                                     "ttft_ms": None if d.ttft_s is None else round(d.ttft_s * 1e3, 3),
                                                     "latency_ms": round(d.latency_s * 1e3, 3)}) + "\n\n"
                    return

            return StreamingResponse(events(), media_type="text/event-stream")
        try:
            fut = server.submit(ids, n_new, body.eos_token_id)
            done = await asyncio.wrap_future(fut)
        except QueueFull as e:
            raise HTTPException(status_code=503, detail=str(e), headers={"Retry-After": "1"})
        except (ValueError, RuntimeError) as e:
            raise HTTPException(status_code=400, detail=str(e))
        out = {"request_id": done.request_id, "output_ids": done.output_ids,
               "ttft_ms": None if done.ttft_s is None else round(done.ttft_s * 1e3, 3),
               "latency_ms": None if done.latency_s is None else round(done.latency_s * 1e3, 3)}
        if tokenizer is not None:
            try:
                out["text"] = tokenizer.decode(done.output_ids)
            except (KeyError, IndexError):      # the model's vocabulary is larger than the tokenizer's
                out["text"] = None
        return out

    return app
