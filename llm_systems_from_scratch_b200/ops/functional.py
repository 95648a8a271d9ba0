"""Numerically-stable functional primitives (softmax family, loss, gradient clipping).

Behavioural parity with the reference's ``llm-core/llm_core/nn_functional.py:8-33``:
max-subtracted softmax / log-softmax, mean next-token cross-entropy over rows, and
global-L2-norm clipping with a 1e-6 guard in the denominator and the coefficient
clamped at one.  The clipping routine here never synchronises with the host: the
coefficient stays a 0-d device tensor.
"""
from __future__ import annotations

from typing import Iterable

import torch


def softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    shifted = x - x.amax(dim=dim, keepdim=True)
    e = shifted.exp()
    return e / e.sum(dim=dim, keepdim=True)


def log_softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    shifted = x - x.amax(dim=dim, keepdim=True)
    return shifted - shifted.exp().sum(dim=dim, keepdim=True).log()


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean negative log-likelihood of ``targets`` (N,) under ``logits`` (N, V)."""
    picked = log_softmax(logits, dim=-1).gather(-1, targets.unsqueeze(-1))
    return -picked.mean()


def global_grad_norm(grads: list[torch.Tensor]) -> torch.Tensor:
    """L2 norm over a list of gradients as a 0-d fp32 tensor on the grads' device."""
    if not grads:
        return torch.zeros(())
    acc = torch.zeros((), dtype=torch.float32, device=grads[0].device)
    for g in grads:
        acc = acc + g.detach().float().pow(2).sum()
    return acc.sqrt()


def clip_gradient(parameters: Iterable[torch.nn.Parameter], max_norm: float) -> torch.Tensor:
    """Scale all gradients in place so their joint L2 norm is at most ``max_norm``.

    Returns the pre-clip norm (0-d tensor).  A model that keeps its gradients in
    one flat arena (see ``models.arena.ParamArena``) is clipped with a single
    sum-of-squares launch and a single scale launch.
    """
    params = list(parameters)
    arena = _common_arena(params)
    if arena is not None:
        return arena.clip_(max_norm)
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return torch.zeros(())
    norm = global_grad_norm(grads)
    coef = torch.clamp(max_norm / (norm + 1e-6), max=1.0)
    for g in grads:
        g.mul_(coef.to(g.dtype))
    return norm


def _common_arena(params):
    """Return the ParamArena that backs *all* of ``params`` (and nothing else), if any."""
    if not params:
        return None
    arena = getattr(params[0], "_arena", None)
    if arena is None or not arena.grads_bound:
        return None
    for p in params:
        if getattr(p, "_arena", None) is not arena:
            return None
    if len(params) != arena.num_tensors:
        return None
    return arena
