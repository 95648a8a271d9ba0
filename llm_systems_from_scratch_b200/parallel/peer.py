"""Peer-memory communicator: hand-written collectives over NVLink / NVSwitch.

Every rank allocates its communication buffers with plain ``cudaMalloc`` (outside PyTorch's caching
allocator), exports them through CUDA IPC, and maps every peer's copy.  torch.distributed is used
only as plumbing (exchanging the 64-byte handles, a few scalar reductions).  The collectives
themselves are kernels of this package (``csrc/comm_kernels.cu``) that load from / store to peer
addresses and synchronise through epoch-numbered flags with bounded waits.

Buffers handed to the collectives must come from ``alloc``; calls on other tensors fall back to
``TorchDistComm`` so the communicator is always usable as a drop-in.

What these replace in the reference: ``dist.all_gather`` of the unit shards
(llm-systems/llm_systems/parallelism/fsdp_zero3.py:131-134), ``dist.reduce_scatter`` + divide + clone followed by the
Triton AdamW (fsdp_zero3.py:172-231, llm-systems/llm_systems/kernels/triton_adamw.py:134-191), the flatten / divide /
``dist.all_reduce`` / unflatten of a DDP bucket (llm-systems/llm_systems/parallelism/ddp.py:20-24) and the parameter
broadcast at construction (ddp.py:57-58).
"""
from __future__ import annotations

import ctypes
import math
import os

import torch
import torch.distributed as dist

from ..ops import native
from .comm import Communicator, TorchDistComm

_ULL = ctypes.c_ulonglong


class _CudaArray:
    """Minimal ``__cuda_array_interface__`` holder so torch can alias raw device memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class ReduceDesc(ctypes.Structure):
    """Mirror of ``B200ReduceDesc`` (csrc/comm_device.cuh): one reduce-scatter of a unit's gradient staging."""
    _fields_ = [("staging", _ULL * 16), ("mc_staging", _ULL), ("flag_bases", _ULL * 16), ("ready_row", _ULL),
                ("done_row", _ULL),
                ("grad_out", ctypes.c_void_p), ("sumsq", ctypes.c_void_p), ("master", ctypes.c_void_p),
                ("m", ctypes.c_void_p), ("v", ctypes.c_void_p), ("mirror", ctypes.c_void_p),
                ("gscale", ctypes.c_void_p), ("lr", ctypes.c_float), ("b1", ctypes.c_float), ("b2", ctypes.c_float),
                ("eps", ctypes.c_float), ("wd", ctypes.c_float), ("alpha_t", ctypes.c_float), ("n", _ULL),
                ("world", ctypes.c_int), ("rank", ctypes.c_int), ("mode", ctypes.c_int), ("epoch", ctypes.c_uint),
                ("limit_ns", _ULL), ("counter", ctypes.c_void_p)]


class GatherDesc(ctypes.Structure):
    """Mirror of ``B200GatherDesc`` (csrc/gemm_tcgen05_2cta.cu): an all-gather carried by a GEMM."""
    _fields_ = [("src", _ULL * 16), ("dst", ctypes.c_void_p), ("shard_bytes", _ULL), ("world", ctypes.c_int),
                ("rank", ctypes.c_int)]


def _declare(lib):
    P, I, L, F = ctypes.c_void_p, ctypes.c_int, _ULL, ctypes.c_float
    U = ctypes.c_uint
    lib.b200_ipc_alloc.argtypes = [L, ctypes.POINTER(_ULL)]
    lib.b200_ipc_free.argtypes = [L]
    lib.b200_ipc_get_handle.argtypes = [L, ctypes.c_char_p]
    lib.b200_ipc_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(_ULL)]
    lib.b200_ipc_close.argtypes = [L]
    lib.b200_peer_barrier.argtypes = [P, L, I, I, U, L, P, P]
    lib.b200_peer_allgather.argtypes = [P, P, L, I, I, I, P]
    lib.b200_peer_reduce_scatter_desc.argtypes = [ctypes.POINTER(ReduceDesc), P, I, P]
    lib.b200_peer_signal.argtypes = [P, L, I, I, U, P]
    lib.b200_peer_wait.argtypes = [P, I, U, L, P, P]
    lib.b200_peer_allreduce.argtypes = [P, P, L, L, L, I, I, U, L, P, P, I, P]
    lib.b200_peer_copy.argtypes = [P, P, L, I, P]
    for n in ("b200_ipc_alloc", "b200_ipc_free", "b200_ipc_get_handle", "b200_ipc_open", "b200_ipc_close",
              "b200_peer_barrier", "b200_peer_allgather", "b200_peer_reduce_scatter_desc", "b200_peer_signal",
              "b200_peer_wait",
              "b200_peer_allreduce", "b200_peer_copy"):
        getattr(lib, n).restype = I


def peer_access_everywhere(world_size: int) -> bool:
    """True when this process's GPU can map the memory of every other GPU of a one-node job of ``world_size`` ranks
    (rank r on device r).  Purely local: no collective, no allocation."""
    if not torch.cuda.is_available() or world_size > torch.cuda.device_count() or world_size > 16:
        return False
    me = torch.cuda.current_device()
    try:
        return all(d == me or torch.cuda.can_device_access_peer(me, d) for d in range(world_size))
    except Exception:
        return False


class PeerComm(Communicator):
    FLAG_ROWS = 1024        # rows of `world` uint32 flags: two per logical buffer (a DDP bucket, an FSDP staging slot)
    ROW_BARRIER = 0
    COUNTER_SLOTS = 256     # CTA counters handed out in turn; a slot is reused only 256 collective launches later
    # A peer that is this late is reported, never waited for indefinitely.  Thirty seconds by default
    # (B200_PEER_WAIT_LIMIT_S): longer than any skew a healthy job produces (first-step set-up, a rank that writes a
    # checkpoint is followed by a host barrier), shorter than the host heartbeat's 60 s.
    WAIT_LIMIT_NS = int(float(os.environ.get("B200_PEER_WAIT_LIMIT_S", "30")) * 1e9)
    GUARD_BYTES = 4096      # canary band before and after every peer-addressable buffer (a multiple of 256)
    GUARD_PATTERN = 0xA5

    def __init__(self, group=None, wait_limit_s: float | None = None, nvls: bool | None = None):
        if not torch.cuda.is_available():
            raise RuntimeError("PeerComm needs CUDA")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)
        if self.world_size > 16:
            raise RuntimeError("PeerComm supports up to 16 ranks on one node")
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.lib = native.load()
        _declare(self.lib)
        self.fallback = TorchDistComm(group)
        self.limit_ns = int((wait_limit_s * 1e9) if wait_limit_s else self.WAIT_LIMIT_NS)
        self.nvls = os.environ.get("B200_NVLS", "0") == "1" if nvls is None else bool(nvls)
        self._allocs: list[dict] = []      # {"base", "nbytes", "peers": [ptr per rank]}
        self._epochs: dict[int, int] = {}
        self._next_row = 2          # row 0: barrier, row 1: "weights published"
        self._rows: dict[str, tuple[int, int]] = {}
        flags = self.alloc(self.FLAG_ROWS * self.world_size, torch.int32)
        self.flags = flags
        self._flag_peers = list(self._find(flags)["peers"])
        self._flag_bases = self._table(self._flag_peers)
        self.launches: dict[str, int] = {}      # peer-memory kernels launched, by kind
        self._counter = torch.zeros(self.COUNTER_SLOTS, dtype=torch.int32, device=self.device)
        self._counter_used = 0
        self.barrier()

    # ------------------------------------------------------------------ memory
    def alloc(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """Collective: a zero-initialised buffer that every peer can address.  All ranks must call
        ``alloc`` in the same order with the same sizes."""
        nbytes = -(-numel * torch.empty((), dtype=dtype).element_size() // 256) * 256
        out = _ULL(0)
        # A guard band on either side of the payload, filled with a pattern that no kernel writes: a peer (or a local
        # kernel) that runs over the end of a staging buffer or a flag row changes it, and ``check_guards`` says so.
        rc = self.lib.b200_ipc_alloc(nbytes + 2 * self.GUARD_BYTES, ctypes.byref(out))
        if rc != 0:
            raise RuntimeError(f"peer buffer allocation of {nbytes} bytes failed ({rc})")
        block = out.value
        bands = torch.as_tensor(_CudaArray(block, nbytes + 2 * self.GUARD_BYTES), device=self.device)
        bands[:self.GUARD_BYTES] = self.GUARD_PATTERN
        bands[self.GUARD_BYTES + nbytes:] = self.GUARD_PATTERN
        torch.cuda.synchronize()
        base = block + self.GUARD_BYTES
        handle = ctypes.create_string_buffer(64)
        if self.lib.b200_ipc_get_handle(block, handle) != 0:
            raise RuntimeError("cudaIpcGetMemHandle failed")
        gathered = [None] * self.world_size
        dist.all_gather_object(gathered, bytes(handle.raw), group=self.group)
        peers = []
        for r, h in enumerate(gathered):
            if r == self.rank:
                peers.append(base)
                continue
            p = _ULL(0)
            rc = self.lib.b200_ipc_open(h, ctypes.byref(p))
            if rc != 0:
                raise RuntimeError(f"cudaIpcOpenMemHandle for rank {r} failed ({rc})")
            peers.append(p.value + self.GUARD_BYTES)
        self._allocs.append({"base": base, "nbytes": nbytes, "peers": peers, "guards": bands})
        raw = torch.as_tensor(_CudaArray(base, nbytes), device=self.device)
        return raw.view(dtype)[:numel]

    def alloc_multicast(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """Collective: like ``alloc``, but the buffer is also bound to an NVLink multicast object (NVLS), so that a
        reduce-scatter can let the NVSwitch add the ranks' copies (``multimem.ld_reduce``) instead of loading every
        peer's copy.  The memory comes from ``torch.distributed._symmetric_memory`` (plumbing: it creates the
        multicast object and exchanges the handles).  Falls back to ``alloc`` when NVLS is off (``B200_NVLS=1`` turns
        it on) or the fabric has no multicast support.  Keep NVLS off in runs where a rank may leave."""
        if not self.nvls:
            return self.alloc(numel, dtype)
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(numel, dtype=dtype, device=self.device)
        t.zero_()
        handle = symm_mem.rendezvous(t, self.group if self.group is not None else dist.group.WORLD)
        mc = int(handle.multicast_ptr or 0)
        ok = torch.tensor([1 if mc else 0], device=self.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) == 0:
            self.nvls = False
            return self.alloc(numel, dtype)
        nbytes = numel * t.element_size()
        self._allocs.append({"base": t.data_ptr(), "nbytes": nbytes, "peers": [int(p) for p in handle.buffer_ptrs],
                             "mc": mc, "keep": (t, handle)})
        torch.cuda.synchronize()
        dist.barrier(group=self.group)        # every rank's buffer is zeroed before anybody reduces over it
        return t

    def check_guards(self) -> None:
        """Raise if any guard band around this rank's peer-addressable buffers was written (one small device
        comparison per buffer and one host read; call it where the host synchronises anyway)."""
        bad = []
        for i, a in enumerate(self._allocs):
            g = a.get("guards")
            if g is None:
                continue
            n = a["nbytes"]
            bad.append(((g[:self.GUARD_BYTES] != self.GUARD_PATTERN).sum()
                        + (g[self.GUARD_BYTES + n:] != self.GUARD_PATTERN).sum()).reshape(1))
        if bad:
            counts = torch.cat(bad).tolist()
            hit = [(i, c) for i, c in enumerate(counts) if c]
            if hit:
                raise RuntimeError(f"rank {self.rank}: guard bytes around peer buffers were overwritten "
                                   f"(buffer index, bytes): {hit}")

    def _find(self, t: torch.Tensor):
        p = t.data_ptr()
        for a in self._allocs:
            if a["base"] <= p < a["base"] + a["nbytes"]:
                return a
        return None

    def _table(self, ptrs: list[int]):
        return (_ULL * self.world_size)(*ptrs)

    def _peer_table(self, t: torch.Tensor):
        a = self._find(t)
        if a is None:
            return None
        off = t.data_ptr() - a["base"]
        return self._table([p + off for p in a["peers"]])

    def _rows_for(self, key: str) -> tuple[int, int]:
        """Two flag rows (ready, done) reserved for one logical buffer."""
        if key not in self._rows:
            if self._next_row + 2 > self.FLAG_ROWS:
                raise RuntimeError("out of flag rows")
            self._rows[key] = (self._next_row, self._next_row + 1)
            self._next_row += 2
        return self._rows[key]

    def _bump(self, row: int) -> int:
        e = self._epochs.get(row, 0) + 1
        self._epochs[row] = e
        return e

    def _counter_slot(self):
        i = self._counter_used % self.COUNTER_SLOTS
        self._counter_used += 1
        return self._counter[i:i + 1]

    def _status(self):
        return native.status_word(self.device).data_ptr()

    @staticmethod
    def _stream():
        return torch.cuda.current_stream().cuda_stream

    # ------------------------------------------------------------- collectives
    def barrier(self):
        """Device-side barrier on the current stream (flag exchange between all ranks)."""
        e = self._bump(self.ROW_BARRIER)
        native._check(self.lib.b200_peer_barrier(self._flag_bases, self.ROW_BARRIER * self.world_size, self.world_size,
                                                 self.rank, e, self.limit_ns, self._status(), self._stream()),
                      "peer_barrier")
        self._count("barrier")

    def pre_gather_sync(self):
        self.barrier()

    ROW_WEIGHTS = 1

    def publish_weights(self):
        """Tell every peer (a flag store from a one-warp kernel on the current stream, no wait) that this rank's
        weight shards are final for the coming step."""
        e = self._bump(self.ROW_WEIGHTS)
        native._check(self.lib.b200_peer_signal(self._flag_bases, self.ROW_WEIGHTS * self.world_size, self.world_size,
                                                self.rank, e, self._stream()), "peer_signal")
        self._count("signal")

    def await_weights(self):
        """Make the current stream wait (bounded) until every peer has published the weights of this step."""
        e = self._epochs.get(self.ROW_WEIGHTS, 0)
        if e == 0:
            return
        flags = self.flags.data_ptr() + self.ROW_WEIGHTS * self.world_size * 4
        native._check(self.lib.b200_peer_wait(flags, self.world_size, e, self.limit_ns, self._status(), self._stream()),
                      "peer_wait")
        self._count("wait")

    def _count(self, kind: str):
        self.launches[kind] = self.launches.get(kind, 0) + 1

    def _ctas(self) -> int:
        """CTAs of a bandwidth kernel: with few peers each thread has few remote loads in flight, so more threads
        are needed to cover the NVLink latency."""
        env = os.environ.get("B200_COMM_CTAS")
        if env:
            return int(env)
        return {2: 296, 4: 192}.get(self.world_size, 128)

    def all_gather(self, full, shard):
        table = self._peer_table(shard)
        nbytes = shard.numel() * shard.element_size()
        if table is None or nbytes % 16 or full.data_ptr() % 16:
            return self.fallback.all_gather(full, shard)
        native._check(self.lib.b200_peer_allgather(table, full.data_ptr(), nbytes, self.world_size, self.rank, self._ctas(),
                                                   self._stream()), "peer_allgather")
        self._count("all_gather")

    def gather_args(self, full, shard):
        """Arguments for a GEMM-carried all-gather of ``shard`` into ``full`` (see ``comm.GatherTask``)."""
        table = self._peer_table(shard)
        nbytes = shard.numel() * shard.element_size()
        if table is None or nbytes % 16 or full.data_ptr() % 16:
            return None
        return table, full.data_ptr(), nbytes, self.world_size, self.rank

    def _reduce_desc(self, staging, key, mode, grad_out, sumsq, adam) -> ReduceDesc:
        """Fill the description of one reduce-scatter and advance the epoch of its flag rows.  Descriptions of one
        ``key`` must be launched in the order in which they were made."""
        a = self._find(staging)
        off = staging.data_ptr() - a["base"]
        ready, done = self._rows_for(key)
        e = self._bump(ready)
        self._epochs[done] = e
        ad = adam or {}
        ptr = lambda t: None if t is None else t.data_ptr()
        d = ReduceDesc()
        for r in range(self.world_size):
            d.staging[r] = a["peers"][r] + off
            d.flag_bases[r] = self._flag_peers[r]
        d.mc_staging = a["mc"] + off if a.get("mc") else 0        # NVLS: the switch adds the copies
        if d.mc_staging:
            self._count("reduce_scatter_nvls")
        d.ready_row, d.done_row = ready * self.world_size, done * self.world_size
        d.grad_out, d.sumsq = ptr(grad_out), ptr(sumsq)
        d.master, d.m, d.v, d.mirror = ptr(ad.get("master")), ptr(ad.get("m")), ptr(ad.get("v")), ptr(ad.get("mirror"))
        d.gscale = ptr(ad.get("gscale"))
        d.lr, d.b1, d.b2 = ad.get("lr", 0.0), ad.get("b1", 0.0), ad.get("b2", 0.0)
        d.eps, d.wd, d.alpha_t = ad.get("eps", 0.0), ad.get("wd", 0.0), ad.get("alpha_t", 0.0)
        d.n = staging.numel() // self.world_size
        d.world, d.rank, d.mode, d.epoch = self.world_size, self.rank, mode, e
        d.limit_ns = self.limit_ns
        d.counter = self._counter_slot().data_ptr()
        return d

    def _launch_reduce(self, desc: ReduceDesc):
        native._check(self.lib.b200_peer_reduce_scatter_desc(ctypes.byref(desc), self._status(), self._ctas(),
                                                             self._stream()), "peer_reduce_scatter")
        self._count("reduce_scatter")

    def _rs_ok(self, out_shard, full) -> bool:
        return (self._find(full) is not None and full.dtype == torch.bfloat16
                and (out_shard is None or out_shard.dtype == torch.float32)
                and (full.numel() // self.world_size) % 8 == 0)

    def reduce_scatter_mean(self, out_shard, full, key: str | None = None, sumsq=None):
        if not self._rs_ok(out_shard, full):
            return self.fallback.reduce_scatter_mean(out_shard, full, sumsq=sumsq)
        self._launch_reduce(self._reduce_desc(full, key or f"rs{full.data_ptr()}", 0, out_shard, sumsq, None))

    def reduce_scatter_adamw(self, full, key, master, m, v, mirror, lr, beta1, beta2, eps, weight_decay, step,
                             grad_scale=None, grad_out=None, sumsq=None):
        """Reduce-scatter fused with the AdamW update of this rank's shard (one kernel)."""
        self._launch_reduce(self._adamw_desc(full, key, master, m, v, mirror, lr, beta1, beta2, eps, weight_decay, step,
                                             grad_scale, grad_out, sumsq))

    def _adamw_desc(self, full, key, master, m, v, mirror, lr, beta1, beta2, eps, weight_decay, step, grad_scale=None,
                    grad_out=None, sumsq=None) -> ReduceDesc:
        alpha_t = lr * math.sqrt(1 - beta2 ** step) / (1 - beta1 ** step)
        return self._reduce_desc(full, key, 1, grad_out, sumsq,
                                 dict(master=master, m=m, v=v, mirror=mirror, gscale=grad_scale, lr=lr, b1=beta1,
                                      b2=beta2, eps=eps, wd=weight_decay, alpha_t=alpha_t))

    def reduce_task(self, full, key, out_shard=None, sumsq=None, adamw: dict | None = None):
        """A reduce-scatter that a later GEMM launch can carry on its copy warps (``ReduceScatterTask``); ``adamw``
        holds the keyword arguments of ``reduce_scatter_adamw`` when the update is to be fused."""
        from .comm import ReduceScatterTask
        if not self._rs_ok(out_shard, full):
            return ReduceScatterTask(lambda: self.fallback.reduce_scatter_mean(out_shard, full, sumsq=sumsq), None)
        if adamw is not None:
            desc = self._adamw_desc(full, key, grad_out=out_shard, sumsq=sumsq, **adamw)
        else:
            desc = self._reduce_desc(full, key, 0, out_shard, sumsq, None)

        def carried():
            self._count("reduce_scatter_carried")
        return ReduceScatterTask(lambda: self._launch_reduce(desc), desc, on_carried=carried)

    def wait_readers(self, staging, key: str | None = None):
        """Before overwriting ``staging``: wait until every peer has finished reading its last contents."""
        key = key or f"rs{staging.data_ptr()}"
        if key not in self._rows:
            return
        _, done = self._rows[key]
        e = self._epochs.get(done, 0)
        if e == 0:
            return
        flags = self.flags.data_ptr() + done * self.world_size * 4
        native._check(self.lib.b200_peer_wait(flags, self.world_size, e, self.limit_ns, self._status(), self._stream()),
                      "peer_wait")
        self._count("wait")

    def all_reduce_mean(self, flat):
        table = self._peer_table(flat)
        if table is None or flat.dtype != torch.float32 or flat.numel() % 4 or flat.data_ptr() % 16:
            return self.fallback.all_reduce_mean(flat)
        ready, done = self._rows_for(f"ar{flat.data_ptr()}:{flat.numel()}")
        e = self._bump(ready)
        self._epochs[done] = e
        native._check(self.lib.b200_peer_allreduce(table, self._flag_bases, ready * self.world_size,
                                                   done * self.world_size, flat.numel(), self.world_size, self.rank, e,
                                                   self.limit_ns, self._counter_slot().data_ptr(), self._status(), 96,
                                                   self._stream()), "peer_allreduce")
        self._count("all_reduce")

    def all_reduce_sum(self, flat):
        self.fallback.all_reduce_sum(flat)      # scalars (norms, counters): plumbing

    BOUNCE_BYTES = 64 << 20
    PEER_BROADCAST = os.environ.get("B200_PEER_BROADCAST", "1") == "1"   # 0: NCCL broadcast instead (init only)

    def broadcast(self, t, src=0):
        """Every rank pulls ``t`` from rank ``src`` through a peer-visible bounce buffer (init-time weights)."""
        if not (t.is_cuda and t.is_contiguous()) or t.numel() == 0 or not self.PEER_BROADCAST:
            return self.fallback.broadcast(t, src)
        if not hasattr(self, "_bounce"):
            self._bounce = self.alloc(self.BOUNCE_BYTES, torch.uint8)    # collective: all ranks broadcast together
        raw = t.view(-1).view(torch.uint8)
        src_ptr = self._find(self._bounce)["peers"][src]
        for off in range(0, raw.numel(), self.BOUNCE_BYTES):
            n = min(self.BOUNCE_BYTES, raw.numel() - off)
            if self.rank == src:
                self._bounce[:n].copy_(raw[off:off + n])
            self.barrier()                  # the source's bounce buffer is complete
            if self.rank != src:
                dst = raw[off:off + n]
                if dst.data_ptr() % 16:
                    tmp = torch.empty(n, dtype=torch.uint8, device=t.device)
                    native._check(self.lib.b200_peer_copy(tmp.data_ptr(), src_ptr, n, 0, self._stream()), "peer_copy")
                    dst.copy_(tmp)
                else:
                    native._check(self.lib.b200_peer_copy(dst.data_ptr(), src_ptr, n, 0, self._stream()), "peer_copy")
            self.barrier()                  # every reader is done before the next chunk overwrites it
