"""Decode-time ops: paged-KV attention and KV-cache append (CUDA kernels, PyTorch statement on CPU).

The reference decodes by running the whole context through the model again for every token
(llm-core/llm_core/model.py:187-236, no KV cache); these ops are what a cached decode step needs instead."""
from __future__ import annotations

import ctypes
import math

import torch

from . import native, torch_impl

_declared = False


def _lib():
    global _declared
    lib = native.load()
    if not _declared:
        P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        lib.b200_paged_decode.argtypes = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, P, P]
        lib.b200_paged_decode.restype = I
        lib.b200_kv_append.argtypes = [P, P, P, P, L, I, L, P, P]
        lib.b200_kv_append.restype = I
        lib.b200_rope_kv_append.argtypes = [P, P, P, P, P, P, L, I, I, I, L, P, P]
        lib.b200_rope_kv_append.restype = I
        _declared = True
    return lib


def kv_append(k_cache, v_cache, qkv, slot_mapping):
    """Write the K and V thirds of qkv (R, 3d) into cache slots ``page * page_size + offset`` (int64, -1 skips)."""
    if not qkv.is_cuda:
        keep = slot_mapping >= 0
        return torch_impl.kv_append(k_cache, v_cache, qkv[keep], slot_mapping[keep])
    lib = _lib()
    d = qkv.shape[1] // 3
    native._req(qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and k_cache.is_contiguous(), "bad kv_append inputs")
    native._req(slot_mapping.dtype == torch.int64 and slot_mapping.numel() == qkv.shape[0], "bad slot mapping")
    native._req(k_cache.shape == v_cache.shape and k_cache.shape[-1] == d, "cache shape does not match qkv")
    num_slots = k_cache.shape[0] * k_cache.shape[1]
    native._check(lib.b200_kv_append(qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), slot_mapping.data_ptr(),
                                     qkv.shape[0], d, num_slots, native.status_word(qkv.device).data_ptr(),
                                     native._stream()), "kv_append")


def rope_kv_append(qkv, cos_sin, positions, k_cache, v_cache, slot_mapping, n_heads: int):
    """Rotate the Q and K thirds of qkv (R, 3d) in place by the angle of ``positions`` and write the rotated K row and
    the V row into cache slot ``slot_mapping`` (-1: rotate only).  One kernel on the GPU; the two separate ops elsewhere."""
    if not qkv.is_cuda:
        from . import rope_ as _rope
        _rope(qkv, cos_sin, positions, n_heads, False, None)
        return kv_append(k_cache, v_cache, qkv, slot_mapping)
    lib = _lib()
    d = qkv.shape[1] // 3
    dh = d // n_heads
    native._req(qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous(),
                "bad rope_kv_append inputs")
    native._req(slot_mapping.dtype == torch.int64 and slot_mapping.numel() == qkv.shape[0], "bad slot mapping")
    native._req(positions.dtype == torch.int32 and positions.numel() == qkv.shape[0] and positions.is_contiguous(),
                "positions must be int32 (R,)")
    native._req(k_cache.shape == v_cache.shape and k_cache.shape[-1] == d, "cache shape does not match qkv")
    native._req(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[0] == 2
                and cos_sin.shape[2] == dh // 2 and dh % 8 == 0, "bad rope cache")
    num_slots = k_cache.shape[0] * k_cache.shape[1]
    native._check(lib.b200_rope_kv_append(qkv.data_ptr(), cos_sin.data_ptr(), positions.data_ptr(), k_cache.data_ptr(),
                                          v_cache.data_ptr(), slot_mapping.data_ptr(), qkv.shape[0], d, dh,
                                          cos_sin.shape[1], num_slots, native.status_word(qkv.device).data_ptr(),
                                          native._stream()), "rope_kv_append")


def choose_splits(rows: int, heads: int, max_context: int, sms: int = 148, head_dim: int = 128) -> int:
    """Context splits per request for the decode kernel (one CTA per (request, split)).

    The CTAs of a launch run in waves of ``sms * resident`` (a CTA has heads * head_dim / 8 threads of 128 registers,
    so two fit on an SM for a 2048-wide model), and a last wave that is mostly empty costs as much as a full one:
    at batch 128 five splits are 2.2 waves (5.6 TB/s measured) where eight are 3.5 (6.1 TB/s).  Among the split
    counts that leave at least 256 tokens per split at full context, take the one whose CTAs fill their waves best;
    ties go to more splits (shorter CTAs, a shorter tail)."""
    threads = max(32, -(-heads * head_dim // 8 // 32) * 32)
    resident = sms * max(1, min(32, 65536 // (128 * threads)))
    best, best_fill = 1, -1.0
    for s in range(1, max(1, min(32, max_context // 256)) + 1):
        ctas = rows * s
        fill = ctas / (-(-ctas // resident) * resident)
        if fill >= best_fill - 1e-9:
            best, best_fill = s, max(fill, best_fill)
    return best


def paged_decode_attention(qkv, k_cache, v_cache, block_tables, context_lens, n_heads: int, splits: int = 0,
                           scratch=None):
    """One query token per request against its paged KV history.

    qkv: (R, 3d) packed (only the query third is read) or (R, d); caches: (num_pages, page_size, d);
    block_tables: (R, max_pages) int32; context_lens: (R,) int32, number of cached tokens to attend to.
    Returns (R, d).  The values inside the tables are checked on the device: a length beyond ``max_pages * page`` or
    a page id beyond the cache is skipped and recorded in the status word (``native.check_status`` raises).
    """
    r, width = qkv.shape
    d = k_cache.shape[-1]
    dh = d // n_heads
    if not qkv.is_cuda:
        return torch_impl.paged_decode_attention(qkv[:, :d], k_cache, v_cache, block_tables, context_lens, n_heads)
    lib = _lib()
    native._req(qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1, "qkv must be bf16 with unit inner stride")
    native._req(block_tables.dtype == torch.int32 and context_lens.dtype == torch.int32, "tables must be int32")
    native._req(block_tables.dim() == 2 and block_tables.is_contiguous() and block_tables.shape[0] >= r
                and context_lens.is_contiguous() and context_lens.numel() >= r, "one table row and one length per request")
    native._req(k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape == v_cache.shape and
                width in (d, 3 * d) and dh * n_heads == d, "cache / query shapes do not match")
    page = k_cache.shape[1]
    max_pages = block_tables.shape[1]
    if splits <= 0:
        splits = choose_splits(r, n_heads, max_pages * page, head_dim=dh)
    out = torch.empty((r, d), dtype=torch.bfloat16, device=qkv.device)
    if scratch is None:
        scratch = torch.empty(r * n_heads * splits * (dh + 2), dtype=torch.float32, device=qkv.device)
    part_o = scratch[:r * n_heads * splits * dh]
    part_ml = scratch[r * n_heads * splits * dh:]
    native._check(lib.b200_paged_decode(qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(),
                                        context_lens.data_ptr(), out.data_ptr(), part_o.data_ptr(), part_ml.data_ptr(),
                                        r, qkv.stride(0), n_heads, dh, page, max_pages, splits, 1.0 / math.sqrt(dh),
                                        k_cache.shape[0], native.status_word(qkv.device).data_ptr(), native._stream()),
                  "paged_decode")
    return out
