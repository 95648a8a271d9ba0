"""Fused-op front end: CUDA tensors go to the hand-written sm_100a kernels, CPU tensors to the
fp32 PyTorch statement of the same op (which is also the test oracle).

There is exactly one GPU code path.  If a tensor lives on a CUDA device and the kernel library
cannot be loaded, the call raises instead of falling back to eager PyTorch.
"""
from __future__ import annotations

import torch

from . import native, torch_impl
from .functional import clip_gradient, cross_entropy, log_softmax, softmax  # noqa: F401


def _dispatch(name):
    cpu_fn = getattr(torch_impl, name)

    def op(first, *args, **kwargs):
        if first.is_cuda:
            return getattr(native, name)(first, *args, **kwargs)
        return cpu_fn(first, *args, **kwargs)

    op.__name__ = name
    op.__doc__ = cpu_fn.__doc__
    return op


gemm = _dispatch("gemm")
rmsnorm_fwd = _dispatch("rmsnorm_fwd")
rmsnorm_bwd = _dispatch("rmsnorm_bwd")
silu_mul_fwd = _dispatch("silu_mul_fwd")
silu_mul_bwd = _dispatch("silu_mul_bwd")
embedding_fwd = _dispatch("embedding_fwd")
embedding_bwd = _dispatch("embedding_bwd")
xent_fwd_bwd = _dispatch("xent_fwd_bwd")
xent_fwd = _dispatch("xent_fwd")
argmax_rows = _dispatch("argmax_rows")
sample_topk = _dispatch("sample_topk")
adamw_step = _dispatch("adamw_step")
sumsq = _dispatch("sumsq")
scale_ = _dispatch("scale_")
cast_copy = _dispatch("cast_copy")


def rope_(qkv, cos_sin, positions, n_heads, inverse=False, seq=None):
    """Rotate Q and K inside packed qkv in place.  ``positions`` (M,) int32 or None with ``seq``."""
    if qkv.is_cuda:
        return native.rope_(qkv, cos_sin, positions, n_heads, inverse, seq)
    if positions is None:
        positions = torch.arange(qkv.shape[0], device=qkv.device) % seq
    return torch_impl.rope_(qkv, cos_sin, positions, n_heads, inverse)


def attention_fwd(qkv, batch, seq, n_heads):
    if qkv.is_cuda:
        from . import attention
        return attention.attention_fwd(qkv, batch, seq, n_heads)
    return torch_impl.attention_fwd(qkv, batch, seq, n_heads)


def attention_bwd(do, qkv, o, lse, batch, seq, n_heads, rope_cache=None):
    """Gradient of packed qkv.  With ``rope_cache`` the Q / K in ``qkv`` are rotated and the result is the
    gradient with respect to the un-rotated projections (inverse rotation fused on the GPU)."""
    if qkv.is_cuda:
        from . import attention
        return attention.attention_bwd(do, qkv, o, lse, batch, seq, n_heads, rope_cache)
    dqkv = torch_impl.attention_bwd(do, qkv, o, lse, batch, seq, n_heads)
    if rope_cache is not None:
        rope_(dqkv, rope_cache, None, n_heads, True, seq)
    return dqkv


def gemm_qkv_rope(x, wqkv, cos_sin, seq, n_heads):
    """QKV projection followed by the rotary embedding on Q and K (one kernel on the GPU when possible)."""
    if x.is_cuda:
        out = native.gemm_qkv_rope(x, wqkv, cos_sin, seq, n_heads)
        if out is not None:
            return out
    qkv = gemm(x, wqkv, "nt")
    rope_(qkv, cos_sin, None, n_heads, False, seq)
    return qkv


def gemm_swiglu(x, wgu, gather=None):
    """Merged gate|up projection and SwiGLU: returns (gu, silu(gate) * up); one kernel on the GPU when possible."""
    if x.is_cuda:
        out = native.gemm_swiglu(x, wgu, gather)
        if out is not None:
            return out
    gu = gemm(x, wgu, "nt", gather=gather)
    return gu, silu_mul_fwd(gu)


def gemm_swiglu_bwd(dy, wdown, gu, gather=None):
    """d(gate | up) for h = silu(gate) * up and dh = dy @ wdown; one kernel on the GPU when possible."""
    if dy.is_cuda:
        out = native.gemm_swiglu_bwd(dy, wdown, gu, gather)
        if out is not None:
            return out
    return silu_mul_bwd(gemm(dy, wdown, "nn", gather=gather), gu)


def clip_coef(sumsq_t, max_norm, coef_out=None, norm_out=None):
    if sumsq_t.is_cuda:
        return native.clip_coef(sumsq_t, max_norm, coef_out, norm_out)
    norm = sumsq_t.sqrt()
    coef = torch.clamp(max_norm / (norm + 1e-6), max=1.0)
    if norm_out is not None:
        norm_out.copy_(norm)
    if coef_out is not None:
        coef_out.copy_(coef)
        return coef_out
    return coef
