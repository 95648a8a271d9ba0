"""Stand-alone autograd wrappers with the per-kernel API of the reference's kernel package.

``TritonRMSNorm`` (reference: llm-systems/llm_systems/kernels/triton_rms_norm.py:240-263),
``triton_silu_mul`` (triton_swiglu.py:95-158) and ``triton_cross_entropy``
(triton_cross_entropy.py:165-197) keep their names because saved ``model_config.json`` files and
user code refer to them; each runs the hand-written sm_100a kernel for bf16 CUDA tensors and the
fp32 PyTorch statement of the same math otherwise.  Like the reference, the loss writes the
gradient over its input logits; unlike it, the loss is accumulated in fp32 and no host
synchronisation happens.
"""
from __future__ import annotations

import torch
from torch import nn

from . import native, torch_impl


def _on_kernel(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).contiguous()
        if _on_kernel(x2) and shape[-1] % 8 == 0:
            w = weight.to(torch.bfloat16).contiguous()
            y, rstd = native.rmsnorm_fwd(x2, w, eps)
        else:
            w = weight
            y, rstd = torch_impl.rmsnorm_fwd(x2, w, eps)
        ctx.save_for_backward(x2, w, rstd)
        ctx.wdtype = weight.dtype
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        dy2 = dy.reshape(x2.shape).contiguous()
        if _on_kernel(x2) and x2.shape[-1] % 8 == 0 and x2.shape[-1] <= 8192:
            dx, dw = native.rmsnorm_bwd(dy2.to(torch.bfloat16), x2, w, rstd)
        else:
            dx, dw = torch_impl.rmsnorm_bwd(dy2, x2, w, rstd)
        return dx.view(dy.shape), dw.to(ctx.wdtype), None


class TritonRMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-5, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, device=device))
        self.eps = eps

    def forward(self, x):
        return _RMSNormFn.apply(x, self.weight, self.eps)

    def extra_repr(self) -> str:
        return f"hidden_size={self.weight.shape[0]}, eps={self.eps}"


class _SiluMulFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        shape = gate.shape
        gu = torch.cat((gate.reshape(-1, shape[-1]), up.reshape(-1, shape[-1])), dim=-1).contiguous()
        ctx.save_for_backward(gu)
        ctx.shape = shape
        if _on_kernel(gu) and shape[-1] % 8 == 0:
            return native.silu_mul_fwd(gu).view(shape)
        return torch_impl.silu_mul_fwd(gu).view(shape)

    @staticmethod
    def backward(ctx, dh):
        (gu,) = ctx.saved_tensors
        f = ctx.shape[-1]
        dh2 = dh.reshape(-1, f).contiguous()
        if _on_kernel(gu) and f % 8 == 0:
            dgu = native.silu_mul_bwd(dh2.to(torch.bfloat16), gu)
        else:
            dgu = torch_impl.silu_mul_bwd(dh2, gu)
        return dgu[:, :f].reshape(ctx.shape), dgu[:, f:].reshape(ctx.shape)


def triton_silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up with a fused forward and backward."""
    return _SiluMulFn.apply(gate, up)


class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, ignore_index):
        rows, v = logits.shape
        need_grad = logits.requires_grad
        if _on_kernel(logits) and logits.stride(1) == 1 and logits.stride(0) % 8 == 0 and logits.data_ptr() % 16 == 0:
            # the kernel works on the row stride, so a column-sliced view of a padded buffer is fine
            buf = torch.as_strided(logits, (rows, logits.stride(0)), (logits.stride(0), 1)) \
                if logits.stride(0) != v else logits
            loss = native.xent_fwd_bwd(buf, targets.contiguous(), 1.0, ignore_index, v, write_grad=need_grad)
            grad = logits
        else:
            work = logits.detach().float().clone()
            loss = torch_impl.xent_fwd_bwd(work, targets, 1.0, ignore_index)
            grad = work.to(logits.dtype)
        if need_grad:
            ctx.save_for_backward(grad)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        (grad,) = ctx.saved_tensors
        return grad * dloss.to(grad.dtype), None, None


def triton_cross_entropy(inputs: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Mean cross-entropy of (N, V) logits; on the kernel path the logits are overwritten by their gradient."""
    return _CrossEntropyFn.apply(inputs, targets, ignore_index)
