"""AdamW with decoupled decay applied after the update, plus the cosine schedule.

Update rule (reference: llm-core/llm_core/optimizer.py:63-82):
    m <- b1 m + (1-b1) g ;  v <- b2 v + (1-b2) g^2
    p <- p - lr * sqrt(1-b2^t)/(1-b1^t) * m / (sqrt(v) + eps)
    p <- p - lr * wd * p                       (decay multiplies the already-updated p)
State per parameter: ``t`` (1 on the first step), ``m``, ``v``.

``AdamW`` is the eager per-tensor optimizer.  ``FusedAdamW`` (reference:
llm-systems/llm_systems/kernels/triton_adamw.py:105-191, which launches once per tensor) updates a
whole flat parameter arena with ONE kernel launch that also rewrites the bf16 compute mirror and
folds in a device-resident gradient-clip coefficient; parameters that do not live in an arena get
one launch each.  Both store ``t = steps + 1`` in their state dict and accept either convention on
load.
"""
from __future__ import annotations

import math
from typing import Callable, Iterable

import torch

from .. import ops


def cosine_lr_schedule(step: int, max_learning_rate: float, min_learning_rate: float, warmup_steps: int,
                       decay_steps: int) -> float:
    """Linear warm-up from 0, cosine decay to the minimum at ``decay_steps``, constant afterwards."""
    if step < warmup_steps:
        return max_learning_rate * step / warmup_steps
    if step > decay_steps:
        return min_learning_rate
    if decay_steps == warmup_steps:
        return min_learning_rate
    progress = (step - warmup_steps) / (decay_steps - warmup_steps)
    return min_learning_rate + 0.5 * (1.0 + math.cos(math.pi * progress)) * (max_learning_rate - min_learning_rate)


def _validate(lr, betas, eps):
    if lr < 0.0:
        raise ValueError(f"Invalid learning rate: {lr}")
    if eps < 0.0:
        raise ValueError(f"Invalid epsilon value: {eps}")
    for i, b in enumerate(betas):
        if not 0.0 <= b < 1.0:
            raise ValueError(f"Invalid beta parameter at index {i}: {b}")


class AdamW(torch.optim.Optimizer):
    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 1e-3, betas: tuple[float, float] = (0.9, 0.95),
                 eps: float = 1e-8, weight_decay: float = 0.01):
        _validate(lr, betas, eps)
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure: Callable | None = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr, (b1, b2), eps, wd = group["lr"], group["betas"], group["eps"], group["weight_decay"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("AdamW does not support sparse gradients")
                st = self.state[p]
                if not st:
                    st["t"] = 1
                    st["m"] = torch.zeros_like(p.grad)
                    st["v"] = torch.zeros_like(p.grad)
                t, g = st["t"], p.grad
                st["m"].mul_(b1).add_(g, alpha=1 - b1)
                st["v"].mul_(b2).addcmul_(g, g, value=1 - b2)
                alpha_t = lr * math.sqrt(1 - b2 ** t) / (1 - b1 ** t)
                p.addcdiv_(st["m"], st["v"].sqrt().add_(eps), value=-alpha_t)
                p.mul_(1 - lr * wd)
                st["t"] = t + 1
        return loss


class FusedAdamW(torch.optim.Optimizer):
    """Single-launch AdamW over flat fp32 state.

    ``set_grad_scale(coef)`` installs a 0-d device tensor that the kernel multiplies into every
    gradient (the clip coefficient), so clipping costs no extra pass over the gradients.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 1e-3, betas: tuple[float, float] = (0.9, 0.95),
                 eps: float = 1e-8, weight_decay: float = 0.01):
        _validate(lr, betas, eps)
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self._grad_scale = None
        self._flat: dict[int, dict] = {}

    def set_grad_scale(self, coef: torch.Tensor | None):
        self._grad_scale = coef

    def _arena_of(self, group):
        params = group["params"]
        arena = getattr(params[0], "_arena", None) if params else None
        if arena is None or len(params) != arena.num_tensors:
            return None
        if any(getattr(p, "_arena", None) is not arena for p in params):
            return None
        return arena

    @torch.no_grad()
    def step(self, closure: Callable | None = None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for gi, group in enumerate(self.param_groups):
            lr, (b1, b2), eps, wd = group["lr"], group["betas"], group["eps"], group["weight_decay"]
            arena = self._arena_of(group)
            if arena is not None and arena.grad is not None:
                if getattr(self, "external_update", False):
                    # the update already ran inside the fused reduce-scatter kernels of this step
                    self.flat_state(gi, group, arena)["t"] += 1
                    arena.mark_mirror(True)
                    continue
                st = self._flat.get(gi)
                if st is None or st["m"].numel() != arena.numel or st["m"].device != arena.master.device:
                    prev_t = st["t"] if st else 1
                    st = {"t": prev_t, "m": torch.zeros_like(arena.master), "v": torch.zeros_like(arena.master)}
                    self._adopt_param_state(group, arena, st)
                    self._flat[gi] = st
                ops.adamw_step(arena.master, arena.grad, st["m"], st["v"], arena.mirror_buffer(), lr, b1, b2, eps, wd,
                               st["t"], self._grad_scale)
                arena.mark_mirror(True)
                st["t"] += 1
                continue
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["t"] = 1
                    st["m"] = torch.zeros_like(p, dtype=torch.float32)
                    st["v"] = torch.zeros_like(p, dtype=torch.float32)
                g = p.grad if p.grad.is_contiguous() else p.grad.contiguous()
                mirror = getattr(p, "_mirror", None)
                if p.is_contiguous() and p.dtype == torch.float32:
                    ops.adamw_step(p.data, g, st["m"], st["v"], mirror, lr, b1, b2, eps, wd, st["t"], self._grad_scale)
                else:
                    tmp = p.data.float().contiguous()
                    ops.adamw_step(tmp, g, st["m"], st["v"], None, lr, b1, b2, eps, wd, st["t"], self._grad_scale)
                    p.data.copy_(tmp)
                st["t"] += 1
        return loss

    def flat_state(self, gi, group, arena):
        """Flat {"t","m","v"} state of group ``gi`` over ``arena`` (created on first use)."""
        st = self._flat.get(gi)
        if st is None or st["m"].numel() != arena.numel:
            st = {"t": 1, "m": torch.zeros_like(arena.master), "v": torch.zeros_like(arena.master)}
            self._adopt_param_state(group, arena, st)
            self._flat[gi] = st
        return st

    # ------------------------------------------------------------- state-dict interchange
    def _adopt_param_state(self, group, arena, flat):
        """Move per-parameter m/v (e.g. loaded from a checkpoint) into the flat buffers."""
        for p, seg in zip(arena.params, arena.segments):
            st = self.state.get(p)
            if st and "m" in st:
                flat["m"][seg.start:seg.start + seg.numel].copy_(st["m"].reshape(-1))
                flat["v"][seg.start:seg.start + seg.numel].copy_(st["v"].reshape(-1))
                flat["t"] = int(st.get("t", flat["t"]))
        for p in arena.params:
            self.state.pop(p, None)

    def state_dict(self):
        """Per-parameter layout {"t","m","v"} identical to the eager optimizer's."""
        for gi, group in enumerate(self.param_groups):
            flat = self._flat.get(gi)
            arena = self._arena_of(group)
            if flat is None or arena is None:
                continue
            for p, seg in zip(arena.params, arena.segments):
                self.state[p] = {"t": flat["t"], "m": flat["m"][seg.start:seg.start + seg.numel].view(seg.shape),
                                 "v": flat["v"][seg.start:seg.start + seg.numel].view(seg.shape)}
        sd = super().state_dict()
        for gi, group in enumerate(self.param_groups):
            if gi in self._flat:
                for p in group["params"]:
                    self.state.pop(p, None)
        return sd

    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        self._flat.clear()   # flat buffers are rebuilt from the per-parameter state on the next step
