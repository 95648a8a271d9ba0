"""ZeRO-3 fully-sharded data parallelism over the fused engine.

Same contract as the reference wrapper (llm-systems/llm_systems/parallelism/fsdp_zero3.py:239-419):
``FSDP(module, process_group=None)`` with ``.module``, ``.fsdp_units``, ``parameters()`` yielding
only the flat shards (so the optimizer state is sharded), ``train/eval/zero_grad``, ``forward`` and
``finish_gradient_synchronization()``; shards are padded with zeros to a multiple of the world size
and rank r owns the r-th slice of its unit.

What is different by design:

* Units are index ranges of the model's flat parameter arena, so sharding, gathering and gradient
  reduction never concatenate or copy per-parameter tensors.  There is one unit per transformer
  block; the reference's single "remaining" unit (fsdp_zero3.py:286-293) is split in two, the
  embedding table and the final norm + lm_head, because they are needed at opposite ends of a step:
  the lm_head gather rides on the last block's forward, its reduce-scatter on the last block's
  backward, and only the embedding's collectives stand alone.
* Parameters are communicated in bf16 (fp32 master, m and v stay sharded); gathered weights land
  in a small pool of persistent buffers that are really reused.
* The block forward/backward is the fused engine.  With the peer-memory communicator the collectives
  of a unit are *carried* by GEMMs of the neighbouring unit: two copy warps in every CTA of the
  tensor-core kernel pull the next unit's weight shards (all-gather) or add up every peer's gradient
  staging of the previous unit (reduce-scatter, optionally with the AdamW update of the shard in the
  same pass) while the MMA warps work.  Other communicators run them on a side stream.
* Gradient clipping through ``clip_gradient(model.parameters(), max_norm)`` uses the *global* norm
  (one all-reduce of a scalar); the reference clips every rank by its local shard norm.
* ``attach_optimizer`` turns on the fused reduce-scatter -> AdamW path (see there for the one-step
  lag of the clip coefficient that it implies).
* With a world size of one, gathered weights alias the shard and gradients are written straight
  into the shard gradient: no copies, no staging.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..models.arena import ParamArena, Segment
from ..models.engine import HeadWeights, block_views
from ..utils.metrics import nvtx_range
from .comm import Communicator, GatherTask, make_communicator


class _ShardArena(ParamArena):
    """Arena over the per-unit shards of one rank: lets AdamW / clipping run as single launches."""

    def __init__(self, units, device, compute_dtype, comm: Communicator, owner):  # noqa: super().__init__ not called
        self.device = device
        self.comm = comm
        self.owner = owner
        self.segments, self.by_name, self.params = [], {}, []
        off = 0
        for u in units:
            seg = Segment(u.name, off, u.shard_numel, (u.shard_numel,))
            self.segments.append(seg)
            self.by_name[u.name] = seg
            off += u.shard_numel
        self.numel = off
        self.num_tensors = len(units)
        self.master = torch.zeros(off, dtype=torch.float32, device=device)
        self.grad = torch.zeros(off, dtype=torch.float32, device=device)
        self.grads_bound = True
        self.compute_dtype = compute_dtype
        if compute_dtype == torch.float32:
            self._mirror = None
        elif hasattr(comm, "alloc"):
            self._mirror = comm.alloc(off, compute_dtype)   # peers pull weight shards straight out of this buffer
        else:
            self._mirror = torch.zeros(off, dtype=compute_dtype, device=device)
        self._mirror_fresh = False
        self._mirror_versions = -1
        self._group_ranges = {}
        self._sumsq = self._coef = self._norm = None
        self.anchor = torch.zeros(1, dtype=torch.float32, device=device, requires_grad=True)

    def grad_sumsq(self) -> torch.Tensor:
        s = super().grad_sumsq()
        self.comm.all_reduce_sum(s)   # global norm: one scalar all-reduce
        return s

    def mark_mirror(self, fresh: bool):
        super().mark_mirror(fresh)
        if fresh:
            self.owner._weights_updated()


class FSDPUnit:
    """One shard group (a transformer block, the embedding table, or the final norm + lm_head)."""

    def __init__(self, owner: "FSDP", index: int, name: str, start: int, end: int, module: nn.Module):
        self.owner, self.index, self.name, self.module = owner, index, name, module
        self.rank, self.world_size = owner.rank, owner.world_size
        self.process_group = owner.process_group
        self.training = True
        self.arena_start, self.arena_end = start, end
        self.original_numel = end - start
        ws = self.world_size
        quantum = ws * 64
        self.padded_numel = -(-self.original_numel // quantum) * quantum
        self.shard_numel = self.padded_numel // ws
        self.flat_shard: nn.Parameter | None = None     # fp32 master shard (bound by the owner)
        self.mirror_shard: torch.Tensor | None = None   # compute-dtype copy that is gathered
        self.flat_full: torch.Tensor | None = None      # gathered weights while resident
        self.full_buf: torch.Tensor | None = None       # dedicated gather buffer (embedding, lm_head units)
        self.stage_buf: torch.Tensor | None = None      # dedicated gradient staging (embedding, lm_head units)
        self.stage_key = None
        self.gather_event = None
        self.scatter_event = None
        self.pending = None
        self.slot = None

    # ---- reference-compatible surface --------------------------------------------------
    def all_gather_params(self, async_op: bool = True):
        self.owner._gather(self)
        if not async_op:
            self.wait_gather()

    def wait_gather(self):
        self.owner._wait_gather(self)

    def discard_full_params(self):
        self.owner._release(self)

    def reduce_scatter_grads(self, comm_stream=None, async_op: bool = True):
        self.owner._reduce_scatter(self)
        if not async_op:
            self.wait_scatter()

    def wait_scatter(self):
        self.owner._wait_scatter(self)


class _FSDPProvider:
    """Feeds the fused engine with gathered weights and gradient staging, driving the collectives."""

    def __init__(self, owner: "FSDP"):
        self.o = owner
        self.arena = owner.shard_arena

    def begin_step(self):
        self.o._begin_step()

    # ---- weights
    def block_weights(self, i: int, backward: bool = False):
        o = self.o
        u = o.layer_units[i]
        if not backward:
            o._wait_gather(u)
            nxt = o.layer_units[i + 1] if i + 1 < len(o.layer_units) else o.lmhead_unit
            o._gather(nxt, defer=True)      # rides on this block's gate|up GEMM
        return o._weight_views(u)

    def embed_weight(self):
        o = self.o
        o._wait_gather(o.embed_unit)
        return o._weight_views(o.embed_unit)

    def head_weights(self, backward: bool = False):
        o = self.o
        o._wait_gather(o.lmhead_unit)
        return o._weight_views(o.lmhead_unit)

    # ---- gradient destinations
    def block_grads(self, i: int):
        return self.o._grad_views(self.o.layer_units[i])

    def embed_grad(self):
        return self.o._grad_views(self.o.embed_unit)

    def head_grads(self):
        return self.o._grad_views(self.o.lmhead_unit)

    # ---- events of the forward / backward pass
    def post_forward(self, kind: str, i: int):
        o = self.o
        if kind == "embed":
            o._release(o.embed_unit)
            return
        keep_last = o.training and torch.is_grad_enabled() and i == len(o.layer_units) - 1
        if not keep_last:   # the last block's weights are needed again first thing in backward
            o._release(o.layer_units[i])

    def pre_backward(self, kind: str, i: int):
        o = self.o
        n = len(o.layer_units)
        if kind == "head":
            if n:
                o._gather(o.layer_units[n - 1])
        elif kind == "block":
            o._gather(o.layer_units[i])
            o._wait_gather(o.layer_units[i])
            if i > 0:
                o._gather(o.layer_units[i - 1], defer=True)

    def take_gather(self, kind: str, i: int):
        task, self.o._deferred = self.o._deferred, None
        return task

    def take_reduce(self, kind: str, i: int):
        task, self.o._deferred_rs = self.o._deferred_rs, None
        return task

    def post_backward(self, kind: str, i: int):
        o = self.o
        if kind == "head":
            o._release(o.lmhead_unit)
            o._reduce_scatter(o.lmhead_unit, defer=bool(o.layer_units))
        elif kind == "block":
            u = o.layer_units[i]
            o._release(u)
            o._reduce_scatter(u, defer=i > 0)
        elif kind == "embed":
            o._reduce_scatter(o.embed_unit)


class FSDP(nn.Module):
    def __init__(self, module: nn.Module, process_group=None, comm: str | Communicator = "auto",
                 fuse_gather: bool | None = None, fuse_reduce: bool | None = None):
        super().__init__()
        if not hasattr(module, "engine"):
            raise TypeError("FSDP wraps a TransformerLM from this package (it drives the fused engine)")
        self.process_group = process_group
        self.comm = comm if isinstance(comm, Communicator) else make_communicator(process_group, comm)
        self.rank, self.world_size = self.comm.rank, self.comm.world_size
        module.use_custom_triton = True   # always run the fused engine under FSDP
        eng = module.engine()
        self.engine_ref = eng
        full = eng.provider.arena
        self.device = full.device
        self.cuda = self.device.type == "cuda"
        self.compute_dtype = full.compute_dtype
        self._by_name = full.by_name
        self._layer_names = eng.provider.layer_names
        self._head_names = eng.provider.head_names
        self._full_segments = full.segments
        self._full_numel = full.numel
        self.comm.broadcast(full.master, src=0)   # every rank shards the same initial weights

        self.fsdp_units: list[FSDPUnit] = []
        self.layer_units: list[FSDPUnit] = []
        for i, layer in enumerate(module.layers):
            s, e = full.group_range(f"layer{i}")
            u = FSDPUnit(self, len(self.fsdp_units), f"layer{i}", s, e, layer)
            self.fsdp_units.append(u)
            self.layer_units.append(u)
        s, e = full.group_range("embed")
        self.embed_unit = FSDPUnit(self, len(self.fsdp_units), "embed", s, e, module.token_embeddings)
        self.fsdp_units.append(self.embed_unit)
        s, e = full.group_range("lmhead")
        self.lmhead_unit = FSDPUnit(self, len(self.fsdp_units), "lmhead", s, e, module.lm_head)
        self.fsdp_units.append(self.lmhead_unit)
        self.unit_modules = [u.module for u in self.fsdp_units]

        self.shard_arena = _ShardArena(self.fsdp_units, self.device, self.compute_dtype, self.comm, self)
        sa = self.shard_arena
        for u, seg in zip(self.fsdp_units, sa.segments):
            lo = u.arena_start + self.rank * u.shard_numel
            hi = min(lo + u.shard_numel, u.arena_end)
            dst = sa.master[seg.start:seg.start + seg.numel]
            if hi > lo:
                dst[:hi - lo].copy_(full.master[lo:hi])
            u.flat_shard = nn.Parameter(dst, requires_grad=True)
            u.flat_shard.grad = sa.grad[seg.start:seg.start + seg.numel]
            u.flat_shard._arena = sa
            u.mirror_shard = (sa._mirror if sa._mirror is not None else sa.master)[seg.start:seg.start + seg.numel]
            sa.params.append(u.flat_shard)
        # release the unsharded weights: module parameters become empty placeholders
        for p in module.parameters():
            p.requires_grad_(False)
            p.data = torch.empty(0, device=p.device, dtype=p.dtype)
            if hasattr(p, "_arena"):
                del p._arena
        full.master = None
        full.grad = None
        full._mirror = None
        eng.provider = _FSDPProvider(self)
        self.module = module

        # ---- persistent communication buffers
        ws = self.world_size
        self.n_slots = 2
        max_p = max((u.padded_numel for u in self.layer_units), default=0)
        if ws > 1:
            mk = lambda n: self._comm_buffer(n)                  # readable by peers
            loc = lambda n: torch.empty(n, dtype=self.compute_dtype, device=self.device)
            self._full_slots = [loc(max_p) for _ in range(self.n_slots)] if max_p else []
            self._stage_slots = [mk(max_p) for _ in range(self.n_slots)] if max_p else []
            for u in (self.embed_unit, self.lmhead_unit):
                u.full_buf = loc(u.padded_numel)
                u.stage_buf = mk(u.padded_numel)
                u.stage_key = f"stage_{u.name}"
        self._slot_owner = [None] * self.n_slots
        self._slot_free_ev = [None] * self.n_slots      # compute stream done with the gathered slot
        self._stage_busy: dict = {}                     # staging key -> event of the stand-alone reduce-scatter
        self._stage_dirty: set = set()                  # staging keys whose readers must be awaited before a rewrite
        self._views_cache: dict = {}
        self._fused_opt = None
        self._max_grad_norm = None
        # A collective that a GEMM of the engine will carry (copy warps inside the tensor-core kernel)
        native_tasks = hasattr(self.comm, "gather_args")
        self.fuse_gather = native_tasks if fuse_gather is None else fuse_gather
        self.fuse_reduce = native_tasks if fuse_reduce is None else fuse_reduce
        self._deferred: GatherTask | None = None
        self._deferred_rs = None          # reduce-scatter waiting for a GEMM of the next backward block
        self._deferred_rs_unit = None
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self._weights_published = False
        self.comm.barrier()      # every rank's buffers exist and its shards are in place before anyone reads them

    # --------------------------------------------------------------------------- helpers
    @property
    def head_unit(self) -> FSDPUnit:
        """The unit holding the final norm and the lm_head (the reference's "remaining" unit also held the
        embedding table, which is ``embed_unit`` here)."""
        return self.lmhead_unit

    def _comm_buffer(self, numel: int) -> torch.Tensor:
        alloc = getattr(self.comm, "alloc_multicast", None) or getattr(self.comm, "alloc", None)
        if alloc is not None:
            return alloc(numel, self.compute_dtype)
        return torch.zeros(numel, dtype=self.compute_dtype, device=self.device)   # the padding behind a unit stays zero

    def _on_comm(self):
        return torch.cuda.stream(self.comm_stream) if self.cuda else _NullCtx()

    def parameters(self, recurse: bool = True):
        for u in self.fsdp_units:
            if u.flat_shard is not None:
                yield u.flat_shard

    def train(self, mode: bool = True):
        self.training = mode
        self.module.train(mode)
        for u in self.fsdp_units:
            u.training = mode
        return self

    def eval(self):
        return self.train(False)

    def zero_grad(self, set_to_none: bool = False):
        pass   # every shard-gradient slice is overwritten by the next backward's reduce-scatter

    # ------------------------------------------------------------------ gather machinery
    def _weights_updated(self):
        """Called (stream-ordered) right after this rank's weight shards were rewritten: tell the peers now, so
        that nobody waits for this rank at the start of the next step longer than necessary."""
        if self.world_size > 1:
            self.comm.publish_weights()
            self._weights_published = True

    def _begin_step(self):
        sa = self.shard_arena
        if sa._mirror is not None:
            ver = sa._versions()
            if not sa._mirror_fresh or ver != sa._mirror_versions:
                ops.cast_copy(sa._mirror, sa.master)
                sa._mirror_fresh, sa._mirror_versions = True, ver
                self._weights_published = False
        if self.world_size > 1:
            if not self._weights_published:
                self.comm.publish_weights()
            self._weights_published = False
            self.comm.await_weights()         # every rank's optimizer has finished rewriting its weight shard
        if self.cuda:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
        self._deferred = None
        if self._deferred_rs is not None:
            self._run_reduce_now(*self._deferred_rs_unit)
        # weights changed since the last gather: drop whatever is still resident
        for u in self.fsdp_units:
            u.flat_full = None
            u.gather_event = None
            u.pending = None
            u.slot = None
        self._slot_owner = [None] * self.n_slots
        if self._fused_opt is not None:
            self._norm_sq.zero_()
        self._gather(self.embed_unit)
        if self.layer_units:
            self._gather(self.layer_units[0])
        else:
            self._gather(self.lmhead_unit)

    def _gather(self, u: FSDPUnit, defer: bool = False):
        if u.flat_full is not None:
            return
        if self.world_size == 1:
            u.flat_full = u.mirror_shard
            return
        if u.full_buf is not None:
            buf, slot = u.full_buf, None
        else:
            slot = u.index % self.n_slots
            buf = self._full_slots[slot][:u.padded_numel]
        if defer and self.fuse_gather:
            # Hand the gather to the engine: its next large GEMM carries it on the compute stream, which is
            # also where the buffer's previous contents were last used, so stream order protects the buffer.
            if self._deferred is not None:
                self._deferred.run()
            task = GatherTask(self.comm, buf[:u.padded_numel], u.mirror_shard)
            self._deferred = task
            u.pending = task
            u.gather_event = None
            u.flat_full = buf[:u.padded_numel]
            u.slot = slot
            if slot is not None:
                self._slot_owner[slot] = u
            return
        with self._on_comm(), nvtx_range(f"fsdp.all_gather.{u.name}"):
            if slot is not None and self._slot_free_ev[slot] is not None:
                self.comm_stream.wait_event(self._slot_free_ev[slot])
            self.comm.all_gather(buf[:u.padded_numel], u.mirror_shard)
            if self.cuda:
                ev = torch.cuda.Event()
                ev.record(self.comm_stream)
                u.gather_event = ev
        u.flat_full = buf[:u.padded_numel]
        u.slot = slot
        if slot is not None:
            self._slot_owner[slot] = u

    def _wait_gather(self, u: FSDPUnit):
        if u.flat_full is None:
            self._gather(u)
        pending = u.pending
        if pending is not None:
            if not pending.done:          # nobody carried it: run it now as a stand-alone collective
                if self._deferred is pending:
                    self._deferred = None
                pending.run()
            u.pending = None
        if u.gather_event is not None:
            torch.cuda.current_stream().wait_event(u.gather_event)
            u.gather_event = None

    def _release(self, u: FSDPUnit):
        if u.flat_full is None or self.world_size == 1:
            if self.world_size == 1:
                u.flat_full = None
            return
        if u.slot is not None and self.cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            self._slot_free_ev[u.slot] = ev
        u.flat_full = None
        u.slot = None

    def _unit_views(self, u: FSDPUnit, buf: torch.Tensor):
        """Tensors of unit ``u`` as views of ``buf`` (element 0 = the unit's first arena element)."""
        if u is self.embed_unit:
            seg = self._by_name[self._head_names["emb"]]
            return buf[seg.start - u.arena_start:seg.start - u.arena_start + seg.numel].view(seg.shape)
        if u is self.lmhead_unit:
            def v(name):
                seg = self._by_name[self._head_names[name]]
                return buf[seg.start - u.arena_start:seg.start - u.arena_start + seg.numel].view(seg.shape)
            return HeadWeights(None, v("norm"), v("lm"))
        return block_views(self._by_name, self._layer_names[u.index], buf, u.arena_start)

    def _weight_views(self, u: FSDPUnit):
        buf = u.flat_full
        key = ("w", u.index, buf.data_ptr())
        v = self._views_cache.get(key)
        if v is None:
            v = self._unit_views(u, buf)
            self._views_cache[key] = v
        return v

    # ---------------------------------------------------------------- gradient machinery
    def _stage_of(self, u: FSDPUnit):
        if u.stage_buf is not None:
            return u.stage_buf[:u.padded_numel], u.stage_key
        slot = u.index % self.n_slots
        return self._stage_slots[slot][:u.padded_numel], f"stage{slot}"

    def _grad_buffer(self, u: FSDPUnit) -> torch.Tensor:
        """Where the backward of ``u`` writes its gradients: the shard gradient itself on one rank, else the unit's
        bf16 staging, once nobody (this rank's last reduce-scatter of it, the peers') still reads the old contents."""
        if self.world_size == 1:
            return u.flat_shard.grad
        stage, key = self._stage_of(u)
        if self._deferred_rs is not None and self._stage_of(self._deferred_rs_unit[1])[1] == key:
            self._run_reduce_now(*self._deferred_rs_unit)     # never wait for readers of a reduce-scatter not yet launched
        ev = self._stage_busy.pop(key, None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        if key in self._stage_dirty:
            self._stage_dirty.discard(key)
            self.comm.wait_readers(stage, key)       # peers are done reading it too
        return stage

    def _grad_views(self, u: FSDPUnit):
        buf = self._grad_buffer(u)
        key = ("g", u.index, buf.data_ptr())
        v = self._views_cache.get(key)
        if v is None:
            v = self._unit_views(u, buf)
            self._views_cache[key] = v
        return v

    def _reduce_task(self, u: FSDPUnit):
        stage, key = self._stage_of(u)
        adamw = None
        if self._fused_opt is not None:
            opt, sa = self._fused_opt, self.shard_arena
            g = opt.param_groups[0]
            st = opt.flat_state(0, g, sa)
            seg = sa.by_name[u.name]
            sl = slice(seg.start, seg.start + seg.numel)
            adamw = dict(master=sa.master[sl], m=st["m"][sl], v=st["v"][sl],
                         mirror=None if sa._mirror is None else sa._mirror[sl], lr=g["lr"], beta1=g["betas"][0],
                         beta2=g["betas"][1], eps=g["eps"], weight_decay=g["weight_decay"], step=st["t"],
                         grad_scale=self._prev_coef if self._max_grad_norm else None)
            return self.comm.reduce_task(stage, key, out_shard=None, sumsq=self._norm_sq, adamw=adamw)
        return self.comm.reduce_task(stage, key, out_shard=u.flat_shard.grad)

    def _reduce_scatter(self, u: FSDPUnit, defer: bool = False):
        """Reduce-scatter the gradient staging of ``u``.  ``defer``: a GEMM of the next backward block carries it
        (compute stream); otherwise it runs now on the communication stream."""
        if self.world_size == 1:
            return
        if self._deferred_rs is not None:          # the previous one found no carrier
            self._run_reduce_now(*self._deferred_rs_unit)
        task = self._reduce_task(u)
        _, key = self._stage_of(u)
        self._stage_dirty.add(key)
        if defer and self.fuse_reduce and task.desc is not None:
            self._deferred_rs = task
            self._deferred_rs_unit = (task, u)
            return
        self._run_reduce_now(task, u)

    def _run_reduce_now(self, task, u: FSDPUnit):
        if self._deferred_rs is task:
            self._deferred_rs = None
        if task.done:
            return
        _, key = self._stage_of(u)
        if self.cuda:
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream())
        with self._on_comm(), nvtx_range(f"fsdp.reduce_scatter.{u.name}"):
            if self.cuda:
                self.comm_stream.wait_event(ready)
            task.run()
            if self.cuda:
                ev = torch.cuda.Event()
                ev.record(self.comm_stream)
                u.scatter_event = ev
                self._stage_busy[key] = ev

    # ------------------------------------------------------- fused reduce-scatter + AdamW
    def attach_optimizer(self, optimizer, max_grad_norm: float | None = None) -> bool:
        """Run AdamW inside each unit's reduce-scatter (one pass over the peers' gradient staging: sum, 1/world
        scale, squared norm, update of the fp32 master / m / v shard and rewrite of the bf16 weight shard; on the
        peer-memory communicator that pass is a single kernel, usually the copy warps of a GEMM).

        The update of a unit then overlaps the backward of the next one and the reduced gradient never goes
        through memory.  Because a unit is updated before the step's global gradient norm exists, clipping uses
        the coefficient computed from the *previous* step's norm (the first step is unclipped);
        ``finish_fused_step()`` after ``finish_gradient_synchronization()`` produces that coefficient, and
        ``optimizer.step()`` only advances the step counter.  Returns False (and changes nothing) on one rank.
        """
        if self.world_size == 1:
            return False
        sa = self.shard_arena
        self._fused_opt = optimizer
        optimizer.external_update = True
        self._max_grad_norm = max_grad_norm
        self._norm_sq = torch.zeros((), dtype=torch.float32, device=self.device)
        self._prev_coef = torch.ones((), dtype=torch.float32, device=self.device)
        self._last_norm = torch.zeros((), dtype=torch.float32, device=self.device)
        optimizer.flat_state(0, optimizer.param_groups[0], sa)
        return True

    def finish_fused_step(self):
        """After ``finish_gradient_synchronization`` in fused mode: turn this step's gradient norm into the clip
        coefficient used by the next step.  Returns the (device) gradient norm of this step."""
        self.comm.all_reduce_sum(self._norm_sq)
        self._last_norm = self._norm_sq.sqrt()
        if self._max_grad_norm:
            ops.clip_coef(self._norm_sq, self._max_grad_norm, self._prev_coef)
        return self._last_norm

    def _wait_scatter(self, u: FSDPUnit):
        if u.scatter_event is not None:
            torch.cuda.current_stream().wait_event(u.scatter_event)
            u.scatter_event = None

    # ---------------------------------------------------------------------- entry points
    def forward(self, token_ids, targets=None):
        """``forward(token_ids)`` returns logits; ``forward(token_ids, targets)`` returns the fused loss."""
        eng = self.engine_ref
        out = eng.logits(token_ids) if targets is None else eng.loss(token_ids, targets)
        if not (self.training and torch.is_grad_enabled()):
            for u in self.fsdp_units:
                self._release(u)
        return out

    def loss(self, token_ids, targets):
        return self.forward(token_ids, targets)

    def finish_gradient_synchronization(self):
        """After ``loss.backward()``: all shard gradients are complete once this returns (stream-ordered)."""
        if self._deferred_rs is not None:
            self._run_reduce_now(*self._deferred_rs_unit)
        if self.cuda and self.world_size > 1:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        for u in self.fsdp_units:
            u.scatter_event = None
            self._release(u)

    # ------------------------------------------------------------------------ checkpoint
    @torch.no_grad()
    def full_state_dict(self, dtype=torch.float32) -> dict:
        """Gather the fp32 master weights of every unit and return a complete (unsharded) state dict
        with the module's own key names.  Collective: call on every rank."""
        flat = torch.zeros(self._full_numel, dtype=torch.float32, device=self.device)
        for u in self.fsdp_units:
            if self.world_size == 1:
                flat[u.arena_start:u.arena_end].copy_(u.flat_shard.data[:u.original_numel])
                continue
            tmp = torch.empty(u.padded_numel, dtype=torch.float32, device=self.device)
            self.comm.all_gather(tmp, u.flat_shard.data)
            flat[u.arena_start:u.arena_end].copy_(tmp[:u.original_numel])
        out = {}
        order = {s.name: s for s in self._full_segments}
        for name, _ in self.module.named_parameters():
            seg = order[name]
            out[name] = flat[seg.start:seg.start + seg.numel].view(seg.shape).to(dtype).cpu()
        return out

    @torch.no_grad()
    def load_full_state_dict(self, state: dict):
        """Inverse of ``full_state_dict``: every rank copies its own slices out of a full state dict."""
        flat = torch.zeros(self._full_numel, dtype=torch.float32, device=self.device)
        order = {s.name: s for s in self._full_segments}
        sd = dict(state)
        self.module._convert_ffn_keys(sd, "")
        for name, seg in order.items():
            flat[seg.start:seg.start + seg.numel].copy_(sd[name].reshape(-1).to(self.device, torch.float32))
        for u in self.fsdp_units:
            lo = u.arena_start + self.rank * u.shard_numel
            hi = min(lo + u.shard_numel, u.arena_end)
            u.flat_shard.data.zero_()
            if hi > lo:
                u.flat_shard.data[:hi - lo].copy_(flat[lo:hi])
        self.shard_arena._mirror_fresh = False


class _NullCtx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
