"""Causal attention on packed QKV: tcgen05 FlashAttention forward/backward wrappers.

qkv is (batch*seq, 3*H*dh) row-major (Q | K | V, heads inside each third); o is (batch*seq, H*dh).
Head sizes 64 and 128 run on the tensor-core kernels; other multiples of 8 up to 128 are zero-padded
to the next supported size around the call (the scale keeps the true head size).

Replaces the reference's attention call (llm-core/llm_core/model.py:381-385: ``scaled_dot_product_attention`` with
``is_causal=True`` on (B, H, S, dh) views, or the explicit softmax(QK^T / sqrt(dh)) V of model.py:308-325 without
``--flash-attn``) and the library backward autograd derives for it.
"""
from __future__ import annotations

import math

import torch

from . import native
from .native import _check, _ptr, _req, _stream


def _pad_heads(t: torch.Tensor, parts: int, n_heads: int, dh: int, dh_pad: int) -> torch.Tensor:
    rows = t.shape[0]
    v = t.view(rows, parts, n_heads, dh)
    out = torch.zeros((rows, parts, n_heads, dh_pad), dtype=t.dtype, device=t.device)
    out[..., :dh] = v
    return out.view(rows, parts * n_heads * dh_pad)


def _unpad_heads(t: torch.Tensor, parts: int, n_heads: int, dh: int, dh_pad: int) -> torch.Tensor:
    rows = t.shape[0]
    return t.view(rows, parts, n_heads, dh_pad)[..., :dh].reshape(rows, parts * n_heads * dh)


def _supported(dh: int) -> int:
    if dh in (64, 128):
        return dh
    _req(dh % 8 == 0 and dh <= 128, "head size must be a multiple of 8 and at most 128")
    return 64 if dh < 64 else 128


def attention_fwd(qkv, batch: int, seq: int, n_heads: int):
    lib = native.load()
    _req(qkv.dtype == torch.bfloat16 and qkv.dim() == 2 and qkv.is_contiguous(), "qkv must be contiguous bf16 2-D")
    rows, three_d = qkv.shape
    _req(rows == batch * seq and three_d % (3 * n_heads) == 0, "qkv shape mismatch")
    d = three_d // 3
    dh = d // n_heads
    dhp = _supported(dh)
    src = qkv if dhp == dh else _pad_heads(qkv, 3, n_heads, dh, dhp)
    o = torch.empty((rows, n_heads * dhp), dtype=qkv.dtype, device=qkv.device)
    lse = torch.empty((batch, n_heads, seq), dtype=torch.float32, device=qkv.device)
    _check(lib.b200_flash_fwd(_ptr(src), _ptr(o), _ptr(lse), batch, seq, n_heads, dhp, 1.0 / math.sqrt(dh),
                              _ptr(native.status_word(qkv.device)), _stream()), "flash_fwd")
    if dhp != dh:
        o = _unpad_heads(o, 1, n_heads, dh, dhp)
    return o, lse


def attention_bwd(do, qkv, o, lse, batch: int, seq: int, n_heads: int, rope_cache=None):
    """dqkv for packed qkv.  With ``rope_cache`` (qkv holds rotated Q / K) the kernels rotate dQ and dK back in
    their epilogues, so no separate inverse-RoPE pass is needed."""
    lib = native.load()
    _req(do.dtype == torch.bfloat16 and do.is_contiguous() and o.is_contiguous(), "do / o must be contiguous bf16")
    rows, three_d = qkv.shape
    d = three_d // 3
    dh = d // n_heads
    dhp = _supported(dh)
    if dhp != dh:
        qkv_p = _pad_heads(qkv, 3, n_heads, dh, dhp)
        do_p = _pad_heads(do, 1, n_heads, dh, dhp)
        o_p = _pad_heads(o, 1, n_heads, dh, dhp)
    else:
        qkv_p, do_p, o_p = qkv, do, o
    dqkv = torch.empty_like(qkv_p)
    delta = torch.empty((batch, n_heads, seq), dtype=torch.float32, device=qkv.device)
    fused = rope_cache is not None and dhp == dh and native.has("b200_flash_bwd_rope")
    if fused:
        _check(lib.b200_flash_bwd_rope(_ptr(qkv_p), _ptr(o_p), _ptr(do_p), _ptr(lse), _ptr(delta), _ptr(dqkv), batch,
                                       seq, n_heads, dhp, 1.0 / math.sqrt(dh), _ptr(rope_cache), rope_cache.shape[1],
                                       _ptr(native.status_word(qkv.device)), _stream()), "flash_bwd")
        return dqkv
    _check(lib.b200_flash_bwd(_ptr(qkv_p), _ptr(o_p), _ptr(do_p), _ptr(lse), _ptr(delta), _ptr(dqkv), batch, seq,
                              n_heads, dhp, 1.0 / math.sqrt(dh), _ptr(native.status_word(qkv.device)), _stream()),
           "flash_bwd")
    if dhp != dh:
        dqkv = _unpad_heads(dqkv, 3, n_heads, dh, dhp)
    if rope_cache is not None:
        native.rope_(dqkv if dqkv.is_contiguous() else dqkv.contiguous(), rope_cache, None, n_heads, True, seq)
    return dqkv


def varlen_attention_fwd(qkv, cu_seqlens, max_seq: int, n_heads: int):
    """Causal attention over packed sequences (prefill): cu_seqlens (n+1,) int32 on the device."""
    lib = native.load()
    _req(qkv.dtype == torch.bfloat16 and qkv.dim() == 2 and qkv.is_contiguous(), "qkv must be contiguous bf16 2-D")
    _req(cu_seqlens.dtype == torch.int32 and cu_seqlens.is_cuda, "cu_seqlens must be int32 on the device")
    rows, three_d = qkv.shape
    d = three_d // 3
    dh = d // n_heads
    dhp = _supported(dh)
    src = qkv if dhp == dh else _pad_heads(qkv, 3, n_heads, dh, dhp)
    o = torch.empty((rows, n_heads * dhp), dtype=qkv.dtype, device=qkv.device)
    _check(lib.b200_flash_varlen_fwd(_ptr(src), _ptr(o), _ptr(cu_seqlens), cu_seqlens.numel() - 1, max_seq, rows,
                                     n_heads, dhp, 1.0 / math.sqrt(dh), _ptr(native.status_word(qkv.device)),
                                     _stream()), "flash_varlen_fwd")
    if dhp != dh:
        o = _unpad_heads(o, 1, n_heads, dh, dhp)
    return o
