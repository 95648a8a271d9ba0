"""Plain-PyTorch statements of every fused op, computed in fp32.

These are (a) the CPU execution path of the engine, so that the hand-written
forward/backward of a transformer block, the sharded optimizer and the wrappers can
be exercised without a GPU, and (b) the oracle that each sm_100a kernel is tested
against.  Each function mirrors the signature of its CUDA twin in ``ops.native``.

Shapes use M = batch * seq rows; activations are row-major ``(M, features)``.
"""
from __future__ import annotations

import math

import torch


def _f(x: torch.Tensor) -> torch.Tensor:
    return x.float()


# ----------------------------------------------------------------------------- GEMM
def gemm(a, b, layout: str, out=None, out_dtype=None, residual=None, accumulate=False, gather=None,
         pad_writable=False, reduce=None, b_stable=False):
    """layout 'nt': a(M,K) b(N,K) -> a@b.T ; 'nn': a(M,K) b(K,N) ; 'tn': a(K,M) b(K,N) -> a.T@b.
    ``gather`` (a pending all-gather that the CUDA kernel would carry) is simply performed first;
    ``pad_writable`` and ``b_stable`` are permissions for the CUDA kernel and change nothing here."""
    if gather is not None:
        gather.run()
    if reduce is not None:
        reduce.run()
    af, bf = _f(a), _f(b)
    if layout == "nt":
        r = af @ bf.t()
    elif layout == "nn":
        r = af @ bf
    elif layout == "tn":
        r = af.t() @ bf
    else:
        raise ValueError(layout)
    if residual is not None:
        r = r + _f(residual)
    dtype = out_dtype or (out.dtype if out is not None else a.dtype)
    if out is not None:
        if accumulate:
            out.add_(r.to(out.dtype))
        else:
            out.copy_(r.to(out.dtype))
        return out
    return r.to(dtype)


# -------------------------------------------------------------------------- RMSNorm
def rmsnorm_fwd(x, w, eps: float):
    xf = _f(x)
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = (xf * rstd) * _f(w)
    return y.to(x.dtype), rstd.squeeze(-1)


def rmsnorm_bwd(dy, x, w, rstd):
    """Returns (dx, dw) for y = x * rstd * w."""
    dyf, xf, wf = _f(dy), _f(x), _f(w)
    r = rstd.unsqueeze(-1)
    g = dyf * wf
    n = x.shape[-1]
    dot = (g * xf).sum(-1, keepdim=True)
    dx = r * g - (r.pow(3) / n) * dot * xf
    dw = (dyf * xf * r).sum(0)
    return dx.to(x.dtype), dw


# --------------------------------------------------------------------------- SwiGLU
def silu_mul_fwd(gu):
    """gu (M, 2F): gate columns first, then up.  Returns silu(gate) * up as (M, F)."""
    f = gu.shape[-1] // 2
    g, u = _f(gu[:, :f]), _f(gu[:, f:])
    return (g * torch.sigmoid(g) * u).to(gu.dtype)


def silu_mul_bwd(dh, gu):
    f = gu.shape[-1] // 2
    g, u, d = _f(gu[:, :f]), _f(gu[:, f:]), _f(dh)
    s = torch.sigmoid(g)
    silu = g * s
    dg = d * u * (s + silu * (1 - s))
    du = d * silu
    return torch.cat([dg, du], dim=-1).to(gu.dtype)


# ----------------------------------------------------------------------------- RoPE
def rope_(qkv, cos_sin, positions, n_heads: int, inverse: bool = False):
    """Rotate the Q and K thirds of qkv (M, 3*H*dh) in place.

    Pairs are adjacent elements (x[2i], x[2i+1]); ``cos_sin`` is (2, ctx, dh/2) fp32;
    ``positions`` is (M,) integer.  ``inverse`` applies the transpose rotation, which
    is what the backward pass needs for dQ and dK.
    """
    m, three_d = qkv.shape
    d = three_d // 3
    dh = d // n_heads
    cos = cos_sin[0][positions.long()]  # (M, dh/2)
    sin = cos_sin[1][positions.long()]
    if inverse:
        sin = -sin
    for part in range(2):
        t = _f(qkv[:, part * d:(part + 1) * d]).reshape(m, n_heads, dh // 2, 2)
        x1, x2 = t[..., 0], t[..., 1]
        c, s = cos.unsqueeze(1), sin.unsqueeze(1)
        r = torch.stack((c * x1 - s * x2, s * x1 + c * x2), dim=-1).reshape(m, d)
        qkv[:, part * d:(part + 1) * d] = r.to(qkv.dtype)
    return qkv


# ------------------------------------------------------------------------ Attention
def attention_fwd(qkv, batch: int, seq: int, n_heads: int):
    """Causal self-attention over packed qkv (B*S, 3*H*dh). Returns o (B*S, H*dh), lse (B,H,S)."""
    m, three_d = qkv.shape
    d = three_d // 3
    dh = d // n_heads
    t = _f(qkv).reshape(batch, seq, 3, n_heads, dh).permute(2, 0, 3, 1, 4)  # (3,B,H,S,dh)
    q, k, v = t[0], t[1], t[2]
    s = (q @ k.transpose(-1, -2)) / math.sqrt(dh)
    mask = torch.ones(seq, seq, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    o = (p @ v).permute(0, 2, 1, 3).reshape(m, d)
    return o.to(qkv.dtype), lse


def attention_bwd(do, qkv, o, lse, batch: int, seq: int, n_heads: int):
    m, three_d = qkv.shape
    d = three_d // 3
    dh = d // n_heads
    t = _f(qkv).reshape(batch, seq, 3, n_heads, dh).permute(2, 0, 3, 1, 4)
    q, k, v = t[0], t[1], t[2]
    dof = _f(do).reshape(batch, seq, n_heads, dh).permute(0, 2, 1, 3)
    of = _f(o).reshape(batch, seq, n_heads, dh).permute(0, 2, 1, 3)
    scale = 1.0 / math.sqrt(dh)
    s = (q @ k.transpose(-1, -2)) * scale
    mask = torch.ones(seq, seq, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.exp(s - lse.unsqueeze(-1))
    dv = p.transpose(-1, -2) @ dof
    dp = dof @ v.transpose(-1, -2)
    delta = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = ds @ k
    dk = ds.transpose(-1, -2) @ q
    out = torch.stack((dq, dk, dv), dim=0).permute(1, 3, 0, 2, 4).reshape(m, three_d)
    return out.to(qkv.dtype)


# ------------------------------------------------------------------------ Embedding
def embedding_fwd(tokens, weight, out_dtype=None):
    return weight[tokens.reshape(-1).long()].to(out_dtype or weight.dtype)


def embedding_bwd(dx, tokens, grad_weight, accumulate=False):
    """Scatter-add rows of dx (M, d) into grad_weight (V, d)."""
    if not accumulate:
        grad_weight.zero_()
    grad_weight.index_add_(0, tokens.reshape(-1).long(), dx.to(grad_weight.dtype))
    return grad_weight


# -------------------------------------------------------------------- Cross entropy
def xent_fwd_bwd(logits, targets, grad_scale: float = 1.0, ignore_index: int = -100, valid_cols=None,
                 loss_out=None, accumulate_loss=False, n_valid=None):
    """Mean CE over non-ignored rows; overwrites ``logits`` with d(loss)/d(logits) * grad_scale.

    ``valid_cols`` limits the vocabulary to the first columns of a padded logits buffer.
    Returns the loss as a 0-d fp32 tensor.
    """
    v = valid_cols or logits.shape[-1]
    lf = _f(logits[:, :v])
    keep = targets != ignore_index
    n = keep.sum().clamp(min=1).float() if n_valid is None else n_valid.float()
    lse = torch.logsumexp(lf, dim=-1)
    tgt = targets.clamp(min=0).long()
    picked = lf.gather(-1, tgt.unsqueeze(-1)).squeeze(-1)
    loss = ((lse - picked) * keep).sum() / n
    p = torch.exp(lf - lse.unsqueeze(-1))
    p.scatter_add_(-1, tgt.unsqueeze(-1), -torch.ones_like(picked).unsqueeze(-1))
    p = p * (keep.unsqueeze(-1) * (grad_scale / n))
    logits[:, :v] = p.to(logits.dtype)
    if v < logits.shape[-1]:
        logits[:, v:] = 0
    if loss_out is not None:
        if accumulate_loss:
            loss_out.add_(loss)
        else:
            loss_out.copy_(loss)
        return loss_out
    return loss


def xent_fwd(logits, targets, ignore_index: int = -100, valid_cols=None, loss_out=None, accumulate_loss=False,
             n_valid=None):
    v = valid_cols or logits.shape[-1]
    lf = _f(logits[:, :v])
    keep = targets != ignore_index
    n = keep.sum().clamp(min=1).float() if n_valid is None else n_valid.float()
    lse = torch.logsumexp(lf, dim=-1)
    picked = lf.gather(-1, targets.clamp(min=0).long().unsqueeze(-1)).squeeze(-1)
    loss = ((lse - picked) * keep).sum() / n
    if loss_out is not None:
        if accumulate_loss:
            loss_out.add_(loss)
        else:
            loss_out.copy_(loss)
        return loss_out
    return loss


# ---------------------------------------------------------------------------- AdamW
def adamw_step(master, grad, m, v, mirror, lr: float, beta1: float, beta2: float, eps: float,
               weight_decay: float, step: int, grad_scale=None):
    """Reference-order AdamW on flat fp32 state (llm-core/llm_core/optimizer.py:63-82).

    ``step`` is the 1-based step count t.  ``grad_scale`` is an optional 0-d tensor
    multiplied into the gradient (the clip coefficient).  Weight decay multiplies the
    already-updated parameter.  ``mirror`` (bf16 copy of the parameter) is refreshed
    when given.
    """
    g = _f(grad)
    if grad_scale is not None:
        g = g * grad_scale.float()
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    alpha_t = lr * math.sqrt(1 - beta2 ** step) / (1 - beta1 ** step)
    master.sub_(alpha_t * m / (v.sqrt() + eps))
    master.sub_(lr * weight_decay * master)
    if mirror is not None:
        mirror.copy_(master)


def sumsq(x, out=None):
    r = _f(x).pow(2).sum()
    if out is not None:
        out.add_(r)
        return out
    return r


def cast_copy(dst, src):
    dst.copy_(src)
    return dst


def scale_(x, coef):
    x.mul_(coef.to(x.dtype) if torch.is_tensor(coef) else coef)
    return x


# --------------------------------------------------------------------- Paged decode
def paged_decode_attention(q, k_cache, v_cache, block_tables, context_lens, n_heads: int):
    """q (R, H*dh); caches (num_pages, page, H*dh); block_tables (R, max_pages) int32;
    context_lens (R,) int32 = number of cached tokens to attend to (inclusive of the new one)."""
    r, d = q.shape
    dh = d // n_heads
    page = k_cache.shape[1]
    out = torch.empty_like(q)
    for i in range(r):
        n = int(context_lens[i])
        npages = (n + page - 1) // page
        pages = block_tables[i, :npages].long()
        k = _f(k_cache[pages]).reshape(-1, n_heads, dh)[:n]
        v = _f(v_cache[pages]).reshape(-1, n_heads, dh)[:n]
        qi = _f(q[i]).reshape(n_heads, dh)
        s = torch.einsum("hd,nhd->hn", qi, k) / math.sqrt(dh)
        p = torch.softmax(s, dim=-1)
        out[i] = torch.einsum("hn,nhd->hd", p, v).reshape(d).to(q.dtype)
    return out


def kv_append(k_cache, v_cache, qkv, slot_mapping):
    """Write the K and V thirds of qkv (R, 3d) into flat cache slots (page*page_size + offset)."""
    d = qkv.shape[1] // 3
    kc = k_cache.view(-1, d)
    vc = v_cache.view(-1, d)
    idx = slot_mapping.long()
    kc[idx] = qkv[:, d:2 * d].to(kc.dtype)
    vc[idx] = qkv[:, 2 * d:].to(vc.dtype)


def varlen_attention_fwd(qkv, cu_seqlens, n_heads: int):
    """Causal attention over several packed sequences; cu_seqlens (n+1,) int32 row offsets."""
    outs = []
    cs = cu_seqlens.tolist()
    for a, b in zip(cs[:-1], cs[1:]):
        o, _ = attention_fwd(qkv[a:b], 1, b - a, n_heads)
        outs.append(o)
    return torch.cat(outs, dim=0)


def argmax_rows(logits, valid_cols=None):
    v = valid_cols or logits.shape[-1]
    return logits[:, :v].float().argmax(dim=-1)


def sample_topk(logits, uniforms, temperature: float, top_k=None, valid_cols=None):
    """Inverse-CDF draw from softmax(logits / temperature) restricted to the top-k logits (ties kept)."""
    x = logits[:, :valid_cols].float() if valid_cols else logits.float()
    if top_k and top_k < x.shape[1]:
        kth = torch.topk(x, top_k, dim=1).values[:, -1:]
        x = x.masked_fill(x < kth, float("-inf"))
    p = torch.softmax(x / temperature, dim=1)
    cdf = p.cumsum(dim=1)
    idx = (cdf <= uniforms.float()[:, None] * cdf[:, -1:]).sum(dim=1)
    return idx.clamp(max=x.shape[1] - 1)
