"""Bucketed data parallelism with gradient all-reduce overlapped with backward.

Contract of the reference wrapper (llm-systems/llm_systems/parallelism/ddp.py:27-99):
``DDP(module, bucket_size_mb=25.0)``, ``.module``, ``forward`` delegating to the module and
``finish_gradient_synchronization()`` to be called between ``backward()`` and ``optimizer.step()``;
rank 0's weights are broadcast at construction; buckets are filled in reverse parameter order and
close once they hold at least ``bucket_size_mb``; gradients are averaged over ranks.

Two execution modes:

* arena mode (a ``TransformerLM`` of this package running the fused engine): gradients already
  live in one flat buffer in backward order, so a bucket is an index range.  As soon as the
  engine reports a block's backward done, the covering bucket is all-reduced *in place* on a side
  stream with the 1/world scale folded into the collective - no flatten, no divide pass, no
  unflatten, and ``param.grad`` keeps pointing at the same memory.
* generic mode (any other ``nn.Module``): per-parameter post-accumulate hooks fill buckets; a full
  bucket is flattened, averaged and all-reduced asynchronously, and views of the reduced buffer are
  installed as ``param.grad`` when synchronisation finishes.
"""
from __future__ import annotations

import torch
from torch import nn

from .comm import Communicator, make_communicator


class GradBucket:
    """Generic-mode bucket: collects parameters whose gradients are ready, reduces when full."""

    def __init__(self, num_params: int, comm: Communicator, stream):
        self.num_params = num_params
        self.comm = comm
        self.stream = stream
        self._params: list[nn.Parameter] = []

    def add_param(self, param: nn.Parameter):
        self._params.append(param)
        if len(self._params) < self.num_params:
            return None
        params, self._params = self._params, []
        flat = torch.cat([p.grad.reshape(-1) for p in params])
        event = None
        if flat.is_cuda:
            ready = torch.cuda.Event()
            ready.record()
            with torch.cuda.stream(self.stream):
                self.stream.wait_event(ready)
                self.comm.all_reduce_mean(flat)
                event = torch.cuda.Event()
                event.record(self.stream)
            flat.record_stream(self.stream)
        else:
            self.comm.all_reduce_mean(flat)
        return event, params, flat


class DDP(nn.Module):
    def __init__(self, module: nn.Module, bucket_size_mb: float = 25.0, process_group=None,
                 comm: str | Communicator = "auto"):
        super().__init__()
        self.module = module
        self.comm = comm if isinstance(comm, Communicator) else make_communicator(process_group, comm)
        self.world_size = self.comm.world_size
        self._bucket_size_bytes = int(bucket_size_mb * 1024 * 1024)
        self._pending: list[tuple] = []
        first = next(module.parameters())
        self._cuda = first.is_cuda
        self.comm_stream = torch.cuda.Stream(device=first.device) if self._cuda else None
        self._arena_mode = bool(getattr(module, "native_supported", lambda: False)())
        if self._arena_mode:
            self._init_arena_buckets()
        else:
            self._init_hook_buckets()

    # ------------------------------------------------------------------------ arena mode
    def _init_arena_buckets(self):
        eng = self.module.engine()
        arena = eng.provider.arena
        self.comm.broadcast(arena.master, src=0)
        arena.mark_mirror(False)
        if hasattr(self.comm, "alloc") and arena.grad is None:
            arena.grad = self.comm.alloc(arena.numel, torch.float32)   # peers reduce it in place over NVLink
        arena.bind_grads()
        n_layers = len(self.module.layers)
        by = arena.by_name
        hn = eng.provider.head_names
        lm, norm, emb = by[hn["lm"]], by[hn["norm"]], by[hn["emb"]]
        align = arena.ALIGN
        pad = lambda seg: seg.start + -(-seg.numel // align) * align
        # events in backward order: ("head", 0), ("block", L-1) ... ("block", 0), ("embed", 0)
        ranges = [(("head", 0), min(norm.start, lm.start), max(pad(norm), pad(lm)))]
        for i in reversed(range(n_layers)):
            s, e = arena.group_range(f"layer{i}")
            ranges.append((("block", i), s, e))
        ranges.append((("embed", 0), emb.start, pad(emb)))
        # merge neighbours (contiguous in the arena) until a bucket reaches the size threshold
        self._arena_buckets: list[dict] = []
        cur = None
        for key, s, e in ranges:
            contiguous = cur is not None and (e == cur["start"] or s == cur["end"])
            if cur is not None and contiguous and (cur["end"] - cur["start"]) * 4 < self._bucket_size_bytes:
                cur["start"], cur["end"] = min(cur["start"], s), max(cur["end"], e)
                cur["last_key"] = key
            else:
                cur = {"start": s, "end": e, "last_key": key}
                self._arena_buckets.append(cur)
        self._fire_on = {b["last_key"]: b for b in self._arena_buckets}
        self._buckets = self._arena_buckets
        self._arena = arena
        eng.provider.post_backward_hooks.append(self._on_backward_event)

    def _on_backward_event(self, kind: str, i: int):
        b = self._fire_on.get((kind, i))
        if b is None or self.world_size == 1:
            return
        flat = self._arena.grad[b["start"]:b["end"]]
        if self._cuda:
            ready = torch.cuda.Event()
            ready.record()
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(ready)
                self.comm.all_reduce_mean(flat)
        else:
            self.comm.all_reduce_mean(flat)

    # ---------------------------------------------------------------------- generic mode
    def _init_hook_buckets(self):
        self._param_to_bucket: dict[nn.Parameter, GradBucket] = {}
        self._buckets: list[GradBucket] = []
        group: list[nn.Parameter] = []
        size = 0

        def close():
            nonlocal group, size
            bucket = GradBucket(len(group), self.comm, self.comm_stream)
            self._buckets.append(bucket)
            for q in group:
                self._param_to_bucket[q] = bucket
            group, size = [], 0

        for p in reversed(list(self.module.parameters())):
            self.comm.broadcast(p.data, src=0)
            if not p.requires_grad:
                continue
            group.append(p)
            size += p.data.nbytes
            p.register_post_accumulate_grad_hook(self._grad_hook)
            if size >= self._bucket_size_bytes:
                close()
        if group:
            close()

    def _grad_hook(self, param: nn.Parameter):
        result = self._param_to_bucket[param].add_param(param)
        if result is not None:
            self._pending.append(result)

    # ----------------------------------------------------------------------------- common
    def forward(self, *inputs, **kwargs):
        return self.module(*inputs, **kwargs)

    def loss(self, token_ids, targets):
        return self.module.loss(token_ids, targets)

    def finish_gradient_synchronization(self):
        if self._arena_mode:
            if self._cuda and self.world_size > 1:
                torch.cuda.current_stream().wait_stream(self.comm_stream)
            return
        for event, params, flat in self._pending:
            if event is not None:
                torch.cuda.current_stream().wait_event(event)
            offset = 0
            for p in params:
                p.grad = flat[offset:offset + p.numel()].view_as(p)
                offset += p.numel()
        self._pending.clear()
