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
        qkv = ops.gemm(h, w.wqkv, "nt", b_stable=True)
        # rotary embedding of Q and K in place and the append of K, V to the paged cache: one kernel on the GPU
        serving_ops.rope_kv_append(qkv, self.rope, positions, self.cache.k[li], self.cache.v[li], slots, cfg.n_heads)
        o = attend(qkv, li)
        x = ops.gemm(o, w.wo, "nt", residual=x, b_stable=True)
        h, _ = ops.rmsnorm_fwd(x, w.n2, cfg.eps)
        gu = ops.gemm(h, w.wgu, "nt", b_stable=True)
        return ops.gemm(ops.silu_mul_fwd(gu), w.wdown, "nt", residual=x, b_stable=True)

    def _logits(self, x):
        h, _ = ops.rmsnorm_fwd(x, self.head.norm, self.cfg.eps)
        buf = torch.empty((x.shape[0], self.cfg.vocab_padded), dtype=x.dtype, device=x.device)
        ops.gemm(h, self.head.lm, "nt", out=buf[:, :self.cfg.vocab], b_stable=True)
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
        ps = self.page_size
        lens = [len(r.prompt) for r in reqs]
        # packed inputs built with numpy (one C loop per request instead of one Python iteration per token)
        tok_np = np.concatenate([np.asarray(r.prompt, dtype=np.int64) for r in reqs])
        pos_np = np.concatenate([np.arange(n, dtype=np.int32) for n in lens])
        slot_np = np.concatenate([np.asarray(r.pages, dtype=np.int64)[np.arange(n) // ps] * ps + np.arange(n) % ps
                                  for r, n in zip(reqs, lens)])
        cu_np = np.zeros(len(reqs) + 1, dtype=np.int32)
        cu_np[1:] = np.cumsum(lens)
        tokens, positions, slots, cu = (torch.from_numpy(a) for a in (tok_np, pos_np, slot_np, cu_np))
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
        st["splits"] = serving_ops.choose_splits(bucket, self.cfg.n_heads, self.max_context,
                                                  head_dim=self.cfg.d_model // self.cfg.n_heads)
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
    # Requests keep one row of the batch arrays for their whole life; the token each row feeds next stays on the
    # device (the decode graph copies its output there), so a decode step can be launched before the previous step's
    # tokens have reached the host.  The host reads them one step behind: while step k + 1 runs on the GPU it appends
    # step k's tokens, retires finished requests and prepares step k + 2.
    def _rows_init(self):
        n = self._bucket(self.max_batch)
        dev = self.device
        self._row_req: list[Request | None] = [None] * n
        self._row_pos = np.full(n, -1, dtype=np.int64)        # position of the token the row feeds next; -1 = idle
        self._row_tab = np.zeros((n, self.max_pages_per_req), dtype=np.int64)
        self._free_rows = list(range(n - 1, -1, -1))
        self._d = {"tokens": torch.zeros(n, dtype=torch.int64, device=dev),
                   "positions": torch.zeros(n, dtype=torch.int32, device=dev),
                   "slots": torch.full((n,), -1, dtype=torch.int64, device=dev),
                   "ctx": torch.ones(n, dtype=torch.int32, device=dev),
                   "tables": torch.zeros((n, self.max_pages_per_req), dtype=torch.int32, device=dev)}
        mk = lambda shape, dt: torch.zeros(shape, dtype=dt, pin_memory=self.cuda)
        # two sets of pinned staging used in turn: a set is refilled only after the step before last has completed
        self._stage = [{"positions": mk(n, torch.int32), "slots": mk(n, torch.int64), "ctx": mk(n, torch.int32),
                        "out": mk(n, torch.int64)} for _ in range(2)]
        self._stage_np = [{k: v.numpy() for k, v in st.items()} for st in self._stage]
        self._tab_host = mk((n, self.max_pages_per_req), torch.int32)
        self._tab_dirty = False
        self._parity = 0
        self._pending: list[tuple] = []
        self._row_graphs: dict[int, dict] = {}

    def _row_graph(self, bucket: int) -> dict:
        g = self._row_graphs.get(bucket)
        if g is not None:
            return g
        d = self._d
        splits = serving_ops.choose_splits(bucket, self.cfg.n_heads, self.max_context,
                                           head_dim=self.cfg.d_model // self.cfg.n_heads)

        def run():
            out = self._decode_body(d["tokens"][:bucket], d["positions"][:bucket], d["slots"][:bucket],
                                    d["tables"][:bucket], d["ctx"][:bucket], splits)
            d["tokens"][:bucket].copy_(out)          # the next step of every row starts from this token
        g = {"run": run}
        if self.use_graphs:
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            keep = d["tokens"][:bucket].clone()
            with torch.cuda.stream(side):            # warm-up outside capture: first-launch set-up happens here
                run()
            torch.cuda.current_stream().wait_stream(side)
            d["tokens"][:bucket].copy_(keep)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                run()
            d["tokens"][:bucket].copy_(keep)         # capture does not execute, but keep the contract obvious
            g["graph"] = graph
        self._row_graphs[bucket] = g
        return g

    def warmup(self):
        """Capture the decode graph of every batch bucket up to ``max_batch`` now, so that no request of a trace pays
        for a capture (a few tenths of a second each) with its time to first token."""
        if not hasattr(self, "_row_req"):
            self._rows_init()
        if self.use_graphs:
            top = self._bucket(self.max_batch)
            for b in self.BUCKETS:
                if b <= top:
                    self._row_graph(b)
            torch.cuda.synchronize()

    def _admit_rows(self, reqs: list[Request], first: torch.Tensor):
        rows = [self._free_rows.pop() for _ in reqs]
        for row, r in zip(rows, reqs):
            self._row_req[row] = r
            r.row = row
            r.issued = 1                                     # the prefill produced the first token
            self._row_pos[row] = len(r.prompt)
            self._row_tab[row, :] = 0
            self._row_tab[row, :len(r.pages)] = r.pages
            if r.issued >= r.max_new_tokens:
                self._row_pos[row] = -1                      # nothing left to decode
        self._tab_host.numpy()[rows] = self._row_tab[rows]
        self._tab_dirty = True
        idx = torch.tensor(rows, dtype=torch.int64)
        if self.cuda:
            idx = idx.pin_memory().to(self.device, non_blocking=True)
        self._d["tokens"].index_copy_(0, idx, first.to(torch.int64))
        self._read_back("prefill", first, list(zip(range(len(reqs)), reqs)))

    def _read_back(self, kind: str, dev_tokens: torch.Tensor, who: list):
        """Queue a device-to-host read of ``dev_tokens``; ``who`` lists (index into it, request)."""
        if self.cuda:
            host = torch.empty(dev_tokens.shape, dtype=torch.int64, pin_memory=True) if kind == "prefill" else \
                self._stage[self._parity]["out"][:dev_tokens.shape[0]]
            host.copy_(dev_tokens, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        else:
            host, ev = dev_tokens.clone(), None
        self._pending.append((kind, ev, host, who))

    def _launch_decode(self) -> int:
        active = np.nonzero(self._row_pos >= 0)[0]
        if active.size == 0:
            return 0
        bucket = self._bucket(int(active[-1]) + 1)
        ps = self.page_size
        st = self._stage_np[self._parity]
        pos = self._row_pos[:bucket]
        live = pos >= 0
        p = np.where(live, pos, 0)
        st["positions"][:bucket] = p
        st["slots"][:bucket] = np.where(live, self._row_tab[np.arange(bucket), p // ps] * ps + p % ps, -1)
        st["ctx"][:bucket] = np.where(live, p + 1, 1)
        d, host = self._d, self._stage[self._parity]
        for name in ("positions", "slots", "ctx"):
            d[name][:bucket].copy_(host[name][:bucket], non_blocking=True)
        if self._tab_dirty:
            d["tables"].copy_(self._tab_host, non_blocking=True)
            self._tab_dirty = False
        g = self._row_graph(bucket)
        if self.use_graphs:
            g["graph"].replay()
        else:
            g["run"]()
        who = [(int(row), self._row_req[row]) for row in active]
        self._read_back("decode", d["tokens"][:bucket], who)
        self._parity ^= 1
        # bookkeeping that needs no token values: positions advance, rows whose last token is now in flight go idle
        self._row_pos[active] += 1
        for row, r in who:
            r.issued += 1
            if r.issued >= r.max_new_tokens:
                self._row_pos[row] = -1
        self.stats["decode_tokens"] += len(who)
        self.stats["decode_steps"] += 1
        return len(who)

    def _finish(self, keep_last: int = 0) -> int:
        """Consume queued read-backs, oldest first, leaving the ``keep_last`` most recent ones in flight."""
        produced = 0
        while len(self._pending) > keep_last:
            kind, ev, host, who = self._pending.pop(0)
            if ev is not None:
                ev.synchronize()
            vals = host.numpy() if host.device.type == "cpu" else host.cpu().numpy()
            t = self._clock()
            for i, r in who:
                if r.t_done is not None:
                    continue                                  # ended by its stop token a step earlier
                r.output.append(int(vals[i]))
                produced += 1
                if kind == "prefill":
                    r.t_first = t
                if r.finished:
                    r.t_done = t
                    row = r.row
                    self._row_pos[row] = -1
                    self._row_req[row] = None
                    self._free_rows.append(row)
                    self.sched.finish(r)
        return produced

    def cancel(self, req: Request) -> bool:
        """Stop ``req`` now: a waiting request leaves the queue, a running one gives its row and its KV pages back and
        keeps the tokens that have reached the host.  Like a stop token, it may have one decode step in flight; that
        step's token is dropped when it is read, and its KV write lands (in stream order) before anything a later owner
        of the pages writes.  Returns False if the request had already finished."""
        if req.t_done is not None:
            return False
        if req in self.sched.waiting:
            self.sched.waiting.remove(req)
            req.t_done = self._clock()
            return True
        if req.row < 0 or self._row_req[req.row] is not req:
            return False
        row = req.row
        req.t_done = self._clock()
        self._row_pos[row] = -1
        self._row_req[row] = None
        self._free_rows.append(row)
        self.sched.finish(req)
        return True

    def step(self, now: float) -> int:
        """One engine iteration at time ``now``: admit + prefill, launch one decode step, then collect the tokens
        of the step before.  Returns the number of tokens that reached the host."""
        if not hasattr(self, "_row_req"):
            self._rows_init()
        admitted = self.sched.admit(now)
        if admitted:
            first = self.prefill(admitted)
            self.sched.start(admitted)
            self._admit_rows(admitted, first)
        launched = self._launch_decode()
        # on the GPU the newest read-back stays in flight while the host goes on; when nothing was launched (every
        # row's last token is already in flight) or without streams, everything is collected now
        return self._finish(keep_last=1 if (self.cuda and launched) else 0)

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
        if not hasattr(self, "_row_req"):
            self._rows_init()
        while not self.sched.idle or self._pending:
            now = self._clock()
            if not self.sched.running and not self._pending:
                nxt = self.sched.next_arrival()
                if realtime and nxt is not None and nxt > now:
                    time.sleep(min(nxt - now, 0.05))
                    continue
            produced = self.step(now)
            if produced == 0 and not self.sched.running and not self._pending and self.sched.waiting:
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
