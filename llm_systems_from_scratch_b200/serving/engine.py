"""Continuous-batching inference engine with a paged KV cache.

New capability relative to the reference, whose only inference path is ``TransformerLM.generate``
(batch 1, no KV cache, llm-core/llm_core/model.py:187-236).  One engine instance drives one GPU;
data-parallel serving runs one replica process per GPU.

Per iteration: newly admitted prompts are packed into one variable-length prefill (FlashAttention
over the packed rows, K/V written straight into the cache pages), then every running request
advances by one token in a single decode step (paged-KV attention).  Decode steps are captured in
CUDA graphs, one per padded batch-size bucket, because at a few milliseconds per step the ~250 kernel
launches of a step would otherwise be launch bound.  Greedy sampling runs on the device.
"""
from __future__ import annotations

import time

import numpy as np
import torch

from .. import ops
from ..ops import serving_ops
from ..utils.metrics import Percentiles
from .kv_cache import PagedKVCache
from .scheduler import Request, Scheduler


class ServingEngine:
    BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)

    def __init__(self, model, num_pages: int | None = None, page_size: int = 16, max_batch: int = 64,
                 max_context: int | None = None, max_prefill_tokens: int = 8192, use_cuda_graphs: bool = True,
                 kv_memory_fraction: float = 0.5):
        model.use_custom_triton = True
        eng = model.engine()
        prov = eng.provider
        prov.begin_step()                       # builds the bf16 weight mirror and its views
        self.cfg = eng.cfg
        self.layers = [prov.block_weights(i) for i in range(self.cfg.n_layers)]
        self.head = prov.head_weights()
        self.rope = eng.rope_cache
        self.device = self.head.emb.device
        self.cuda = self.device.type == "cuda"
        self.dtype = self.head.emb.dtype
        self.max_context = min(max_context or model.context_length, self.rope.shape[1])
        self.page_size = page_size
        self.max_pages_per_req = -(-self.max_context // page_size)
        if num_pages is None:
            per_page = PagedKVCache.bytes_per_page(self.cfg.n_layers, self.cfg.d_model, page_size,
                                                   2 if self.dtype == torch.bfloat16 else 4)
            if self.cuda:
                free, _ = torch.cuda.mem_get_info(self.device)
                num_pages = max(self.max_pages_per_req * 2, int(free * kv_memory_fraction) // per_page)
                num_pages = min(num_pages, self.max_pages_per_req * max_batch + 8)
            else:
                num_pages = self.max_pages_per_req * max_batch
        self.cache = PagedKVCache(self.cfg.n_layers, self.cfg.d_model, num_pages, page_size, self.device, self.dtype)
        self.sched = Scheduler(self.cache.allocator, page_size, max_batch, max_prefill_tokens, self.max_context)
        self.max_batch = max_batch
        self.use_graphs = use_cuda_graphs and self.cuda
        self._graphs: dict[int, dict] = {}
        try:
            from ..utils import host_runtime
            self._host_rt = host_runtime if host_runtime.available() else None
        except Exception:
            self._host_rt = None
        self._temperature, self._top_k = 0.0, None
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "decode_steps": 0, "prefill_steps": 0}

    # ------------------------------------------------------------------ model pieces
    def _block(self, x, w, li: int, positions, slots, attend):
        cfg = self.cfg
        h, _ = ops.rmsnorm_fwd(x, w.n1, cfg.eps)
        qkv = ops.gemm(h, w.wqkv, "nt")
        ops.rope_(qkv, self.rope, positions, cfg.n_heads, False, None)
        serving_ops.kv_append(self.cache.k[li], self.cache.v[li], qkv, slots)
        o = attend(qkv, li)
        x = ops.gemm(o, w.wo, "nt", residual=x)
        h, _ = ops.rmsnorm_fwd(x, w.n2, cfg.eps)
        gu = ops.gemm(h, w.wgu, "nt")
        return ops.gemm(ops.silu_mul_fwd(gu), w.wdown, "nt", residual=x)

    def _logits(self, x):
        h, _ = ops.rmsnorm_fwd(x, self.head.norm, self.cfg.eps)
        buf = torch.empty((x.shape[0], self.cfg.vocab_padded), dtype=x.dtype, device=x.device)
        ops.gemm(h, self.head.lm, "nt", out=buf[:, :self.cfg.vocab])
        return buf

    def _greedy(self, logits_buf):
        """Next token per row: argmax, or a draw from softmax(logits / temperature) over the top-k logits when
        ``set_sampling`` asked for one (one kernel on the GPU: filter, softmax and inverse-CDF draw, no sort)."""
        if self._temperature == 0:
            return ops.argmax_rows(logits_buf, self.cfg.vocab)
        rows = logits_buf.shape[0]
        if logits_buf.is_cuda and logits_buf.dtype == torch.bfloat16:
            u = torch.rand(rows, device=logits_buf.device)
            return ops.sample_topk(logits_buf, u, self._temperature, self._top_k, self.cfg.vocab)
        last = logits_buf[:, :self.cfg.vocab].float() / self._temperature
        if self._top_k:
            kth = torch.topk(last, min(self._top_k, last.shape[-1])).values[:, -1:]
            last = last.masked_fill(last < kth, float("-inf"))
        return torch.multinomial(torch.softmax(last, dim=-1), 1).reshape(-1)

    def set_sampling(self, temperature: float = 0.0, top_k: int | None = None):
        """temperature 0 = greedy.  Decode graphs captured under another setting are dropped."""
        if (temperature, top_k) != (self._temperature, self._top_k):
            self._temperature, self._top_k = float(temperature), top_k
            self._graphs.clear()

    # ------------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, reqs: list[Request]) -> torch.Tensor:
        """Run the prompts of ``reqs`` (pages already reserved); returns their first generated tokens."""
        lens = [len(r.prompt) for r in reqs]
        tokens = torch.tensor([t for r in reqs for t in r.prompt], dtype=torch.int64)
        positions = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens])
        slots = torch.tensor([s for r in reqs for s in self.cache.slots(r.pages, 0, len(r.prompt))], dtype=torch.int64)
        cu = torch.zeros(len(reqs) + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(lens).cumsum(0)
        last = (cu[1:] - 1).long()
        if self.cuda:
            tokens, positions, slots, cu_d, last = (t.pin_memory().to(self.device, non_blocking=True)
                                                    for t in (tokens, positions, slots, cu, last))
        else:
            cu_d = cu
        max_len = max(lens)

        def attend(qkv, li):
            if qkv.is_cuda:
                from ..ops import attention
                return attention.varlen_attention_fwd(qkv, cu_d, max_len, self.cfg.n_heads)
            return ops.torch_impl.varlen_attention_fwd(qkv, cu, self.cfg.n_heads)

        x = ops.embedding_fwd(tokens, self.head.emb)
        for li, w in enumerate(self.layers):
            x = self._block(x, w, li, positions, slots, attend)
        first = self._greedy(self._logits(x[last].contiguous()))
        self.stats["prefill_tokens"] += sum(lens)
        self.stats["prefill_steps"] += 1
        return first

    # ------------------------------------------------------------------------- decode
    def _decode_body(self, tokens, positions, slots, tables, ctx_lens, splits):
        def attend(qkv, li):
            return serving_ops.paged_decode_attention(qkv, self.cache.k[li], self.cache.v[li], tables, ctx_lens,
                                                      self.cfg.n_heads, splits)
        x = ops.embedding_fwd(tokens, self.head.emb)
        for li, w in enumerate(self.layers):
            x = self._block(x, w, li, positions, slots, attend)
        return self._greedy(self._logits(x))

    def _bucket(self, n: int) -> int:
        for b in self.BUCKETS:
            if b >= n:
                return b
        return n

    def _graph_for(self, bucket: int) -> dict:
        g = self._graphs.get(bucket)
        if g is not None:
            return g
        dev = self.device
        st = {"tokens": torch.zeros(bucket, dtype=torch.int64, device=dev),
              "positions": torch.zeros(bucket, dtype=torch.int32, device=dev),
              "slots": torch.full((bucket,), -1, dtype=torch.int64, device=dev),
              "tables": torch.zeros((bucket, self.max_pages_per_req), dtype=torch.int32, device=dev),
              "ctx": torch.ones(bucket, dtype=torch.int32, device=dev)}
        st["splits"] = serving_ops.choose_splits(bucket, self.cfg.n_heads, self.max_context)
        run = lambda: self._decode_body(st["tokens"], st["positions"], st["slots"], st["tables"], st["ctx"], st["splits"])
        if self.use_graphs:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):            # warm-up outside capture: first-launch set-up happens here
                run()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                st["out"] = run()
            st["graph"] = graph
        st["run"] = run
        self._graphs[bucket] = st
        return st

    @torch.no_grad()
    def decode(self, reqs: list[Request]) -> list[int]:
        """Advance every request in ``reqs`` by one token; returns the new tokens (host ints)."""
        n = len(reqs)
        bucket = self._bucket(n)
        st = self._graph_for(bucket)
        ps = self.page_size
        # Host staging is pinned once per bucket and refilled in place through numpy views (the previous step ended
        # with a device-to-host read, so no copy from these buffers is still in flight).
        host = st.get("host")
        if host is None:
            mk = lambda shape, dt: torch.zeros(shape, dtype=dt, pin_memory=self.cuda)
            host = st["host"] = {"tokens": mk(bucket, torch.int64), "positions": mk(bucket, torch.int32),
                                 "slots": mk(bucket, torch.int64), "ctx": mk(bucket, torch.int32),
                                 "tables": mk((bucket, self.max_pages_per_req), torch.int32)}
            st["host_np"] = {k: v.numpy() for k, v in host.items()}
        hn = st["host_np"]
        p = np.fromiter((r.context_len - 1 for r in reqs), dtype=np.int64, count=n)   # position of the token being fed
        hn["tokens"][:n] = np.fromiter((r.output[-1] for r in reqs), dtype=np.int64, count=n)
        hn["tokens"][n:] = 0
        hn["positions"][:n] = p
        hn["positions"][n:] = 0
        hn["slots"][:n] = np.fromiter((r.pages[q // ps] for r, q in zip(reqs, p)), dtype=np.int64, count=n) * ps + p % ps
        hn["slots"][n:] = -1
        hn["ctx"][:n] = p + 1
        hn["ctx"][n:] = 1
        if self._host_rt is not None:
            self._host_rt.block_table_into([r.pages for r in reqs], host["tables"], 0)
        else:
            tb = hn["tables"]
            tb[:] = 0
            for i, r in enumerate(reqs):
                tb[i, :len(r.pages)] = r.pages
        for name in ("tokens", "positions", "slots", "ctx", "tables"):
            st[name].copy_(host[name], non_blocking=True)
        if self.use_graphs:
            st["graph"].replay()
            out = st["out"]
        else:
            out = st["run"]()
        new = out[:n].tolist()
        self.stats["decode_tokens"] += n
        self.stats["decode_steps"] += 1
        return new

    # ---------------------------------------------------------------------- main loop
    def step(self, now: float) -> int:
        """One engine iteration at time ``now``: admit + prefill, then one decode step.  Returns the
        number of tokens produced."""
        produced = 0
        admitted = self.sched.admit(now)
        if admitted:
            first = self.prefill(admitted).tolist()
            t = self._clock()
            for r, tok in zip(admitted, first):
                r.output.append(int(tok))
                r.t_first = t
            self.sched.start(admitted)
            produced += len(admitted)
            self.sched.retire(t)
        if self.sched.running:
            batch = list(self.sched.running)
            for r, tok in zip(batch, self.decode(batch)):
                r.output.append(int(tok))
            produced += len(batch)
            self.sched.retire(self._clock())
        return produced

    def _clock(self) -> float:
        return time.perf_counter() - self._t0 if self._realtime else self._virtual

    def run(self, requests: list[Request], realtime: bool = True) -> dict:
        """Replay ``requests`` (sorted by arrival).  ``realtime`` honours arrival times against the wall
        clock; otherwise every request counts as already arrived (offline throughput)."""
        self._realtime = realtime
        self._virtual = float("inf")
        for r in sorted(requests, key=lambda q: q.arrival):
            self.sched.add(r)
        if self.cuda:
            torch.cuda.synchronize()
        self._t0 = time.perf_counter()
        while not self.sched.idle:
            now = self._clock()
            if not self.sched.running:
                nxt = self.sched.next_arrival()
                if realtime and nxt is not None and nxt > now:
                    time.sleep(min(nxt - now, 0.05))
                    continue
            produced = self.step(now)
            if produced == 0 and not self.sched.running and self.sched.waiting:
                head = self.sched.waiting[0]
                if not realtime or head.arrival <= now:
                    # nothing runs, so every page is free, and the oldest arrived request still was not admitted
                    raise RuntimeError(f"request {head.rid} does not fit in the KV cache")
        if self.cuda:
            torch.cuda.synchronize()
        wall = time.perf_counter() - self._t0
        return self.summarise(requests, wall)

    def summarise(self, requests: list[Request], wall: float) -> dict:
        ttft, lat = Percentiles(), Percentiles()
        out_tokens = 0
        for r in requests:
            out_tokens += len(r.output)
            if r.t_first is not None and self._realtime:
                ttft.add(r.t_first - r.arrival)
            if r.t_done is not None and self._realtime:
                lat.add(r.t_done - r.arrival)
        return {"requests": len(requests), "output_tokens": out_tokens, "wall_s": wall,
                "decode_tok_per_s": out_tokens / wall if wall > 0 else float("nan"),
                "prefill_tokens": self.stats["prefill_tokens"], "decode_steps": self.stats["decode_steps"],
                "ttft_p50_s": ttft.pct(50), "ttft_p99_s": ttft.pct(99), "latency_p50_s": lat.pct(50),
                "kv_pages": self.cache.num_pages, "kv_occupancy_end": self.cache.occupancy()}

    def generate(self, prompts: list[list[int]], max_new_tokens: int, eos_token_id: int | None = None,
                 temperature: float = 0.0, top_k: int | None = None) -> list[list[int]]:
        """Offline batched generation through the continuous-batching loop (greedy unless a temperature is given).
        An end-of-sequence token ends a request and is part of its output."""
        self.set_sampling(temperature, top_k)
        reqs = [Request(i, list(p), max_new_tokens, 0.0, eos_token_id) for i, p in enumerate(prompts)]
        self.run(reqs, realtime=False)
        return [r.output for r in reqs]
