"""Flat parameter arena: one fp32 master buffer, one bf16 compute mirror, one gradient buffer.

The reference keeps every parameter as its own tensor, so its optimizer launches one kernel
per tensor (llm-systems/llm_systems/kernels/triton_adamw.py:147-189), its DDP wrapper
flattens and unflattens gradients around every all-reduce (llm-systems/llm_systems/
parallelism/ddp.py:20-24,90-99) and its FSDP wrapper concatenates them before every
reduce-scatter (llm-systems/llm_systems/parallelism/fsdp_zero3.py:182-189).  Here the model's
``nn.Parameter`` objects are *views* into one contiguous buffer laid out so that tensors
which are consumed together sit together (q|k|v rows, gate|up rows).  Consequences:

* the fused QKV and gate/up GEMMs read one weight matrix without any concatenation;
* AdamW, gradient-norm and clipping are single launches over the whole model;
* a DDP bucket or an FSDP unit is just an index range, never a copy.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from .. import ops


@dataclass
class Segment:
    name: str          # qualified parameter name in the model
    start: int         # element offset in the arena
    numel: int
    shape: tuple


class ParamArena:
    ALIGN = 64  # elements; keeps every tensor 128-byte aligned in bf16 and 256-byte aligned in fp32

    def __init__(self, ordered: list[tuple[str, nn.Parameter]], groups: list[tuple[str, int, int]] | None = None):
        """``ordered``: (name, parameter) pairs in arena order.  ``groups``: optional named index
        ranges over ``ordered`` (e.g. one per transformer layer) exposed as ``group_range``."""
        device = ordered[0][1].device
        self.device = device
        self.segments: list[Segment] = []
        self.by_name: dict[str, Segment] = {}
        off = 0
        for name, p in ordered:
            seg = Segment(name, off, p.numel(), tuple(p.shape))
            self.segments.append(seg)
            self.by_name[name] = seg
            off += -(-p.numel() // self.ALIGN) * self.ALIGN
        self.numel = off
        self.num_tensors = len(ordered)
        self.master = torch.zeros(off, dtype=torch.float32, device=device)
        self.params = [p for _, p in ordered]
        for seg, p in zip(self.segments, self.params):
            view = self.master[seg.start:seg.start + seg.numel].view(seg.shape)
            view.copy_(p.data)
            p.data = view
            p._arena = self
        self._group_ranges: dict[str, tuple[int, int]] = {}
        for gname, first, last in (groups or []):
            s = self.segments[first].start
            e_seg = self.segments[last]
            e = e_seg.start + (-(-e_seg.numel // self.ALIGN) * self.ALIGN)
            self._group_ranges[gname] = (s, e)
        self.compute_dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
        self._mirror: torch.Tensor | None = None
        self._mirror_fresh = False
        self._mirror_versions = -1
        self.grad: torch.Tensor | None = None
        self.grads_bound = False
        self._sumsq = None
        self._coef = None
        self._norm = None
        # Anchor that makes autograd call the engine's backward functions.
        self.anchor = torch.zeros(1, dtype=torch.float32, device=device, requires_grad=True)

    # ---------------------------------------------------------------- compute mirror
    def _versions(self) -> int:
        # In-place PyTorch updates of a parameter (optimizers, load_state_dict) bump its version
        # counter; kernels launched through raw pointers do not and report freshness explicitly.
        return sum(p._version for p in self.params)

    def mirror(self) -> torch.Tensor:
        """bf16 copy of the master weights (the master itself on CPU), refreshed when stale."""
        if self.compute_dtype == torch.float32:
            return self.master
        if self._mirror is None:
            self._mirror = torch.empty(self.numel, dtype=torch.bfloat16, device=self.device)
            self._mirror_fresh = False
        ver = self._versions()
        if not self._mirror_fresh or ver != self._mirror_versions:
            ops.cast_copy(self._mirror, self.master)
            self._mirror_fresh = True
            self._mirror_versions = ver
        return self._mirror

    def mirror_buffer(self) -> torch.Tensor | None:
        """The raw mirror storage for an optimizer that rewrites it in the update kernel."""
        if self.compute_dtype == torch.float32:
            return None
        if self._mirror is None:
            self._mirror = torch.empty(self.numel, dtype=torch.bfloat16, device=self.device)
        return self._mirror

    def mark_mirror(self, fresh: bool):
        """Called by an optimizer that updated master and mirror together in one kernel."""
        self._mirror_fresh = fresh
        self._mirror_versions = self._versions()

    # --------------------------------------------------------------------- gradients
    def ensure_grads(self) -> torch.Tensor:
        if self.grad is None:
            self.grad = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
        return self.grad

    def bind_grads(self):
        """Point every parameter's ``.grad`` at its slice of the flat gradient buffer."""
        g = self.ensure_grads()
        for seg, p in zip(self.segments, self.params):
            view = g[seg.start:seg.start + seg.numel].view(seg.shape)
            if p.grad is None or p.grad.data_ptr() != view.data_ptr():
                p.grad = view
        self.grads_bound = True

    def view(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        seg = self.by_name[name]
        return flat[seg.start:seg.start + seg.numel].view(seg.shape)

    def group_range(self, gname: str) -> tuple[int, int]:
        return self._group_ranges[gname]

    # ---------------------------------------------------------------------- clipping
    def grad_sumsq(self) -> torch.Tensor:
        if self._sumsq is None:
            self._sumsq = torch.zeros((), dtype=torch.float32, device=self.device)
        self._sumsq.zero_()
        ops.sumsq(self.ensure_grads(), self._sumsq)
        return self._sumsq

    def clip_coef(self, max_norm: float) -> torch.Tensor:
        """Device-resident clip coefficient for the current gradients; nothing is scaled."""
        if self._coef is None:
            self._coef = torch.ones((), dtype=torch.float32, device=self.device)
            self._norm = torch.zeros((), dtype=torch.float32, device=self.device)
        ops.clip_coef(self.grad_sumsq(), max_norm, self._coef, self._norm)
        return self._coef

    def clip_(self, max_norm: float) -> torch.Tensor:
        coef = self.clip_coef(max_norm)
        ops.scale_(self.grad, coef)
        return self._norm
