"""Hand-written forward and backward of the decoder stack on fused ops.

Instead of letting autograd record ~60 small kernels per block (the reference's eager path,
llm-core/llm_core/model.py:289-292,353-390), each transformer block is ONE autograd node whose
forward and backward are explicit sequences of fused kernels:

    forward : rmsnorm -> QKV GEMM -> RoPE -> flash attention -> out-proj GEMM (+residual)
              rmsnorm -> gate|up GEMM -> silu*mul -> down GEMM (+residual)
    backward: the mirrored 7 dgrad / wgrad GEMMs, attention backward, fused norm backward.

Weights reach a block through a *provider*, so the same code serves a locally held arena, a
DDP replica (provider fires bucket all-reduces as ranges of the gradient arena complete) and
FSDP (provider hands out gathered bf16 shards and reduce-scatters the gradient staging).
Activations are row-major ``(batch*seq, features)``; attention reads Q, K and V straight out of
the packed QKV activation, so no head transposes exist anywhere.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import NamedTuple

import torch

from .. import ops
from ..utils.metrics import nvtx_range


class BlockWeights(NamedTuple):
    wqkv: torch.Tensor   # (3d, d)
    wo: torch.Tensor     # (d, d)
    wgu: torch.Tensor    # (2F, d)  gate rows, then up rows
    wdown: torch.Tensor  # (d, F)
    n1: torch.Tensor     # (d,)
    n2: torch.Tensor     # (d,)


class HeadWeights(NamedTuple):
    emb: torch.Tensor    # (V, d)
    norm: torch.Tensor   # (d,)
    lm: torch.Tensor     # (V, d)


@dataclass
class EngineConfig:
    d_model: int
    n_heads: int
    d_ff: int
    vocab: int
    n_layers: int
    eps: float = 1e-5
    recompute: bool = False   # per-block activation checkpointing

    @property
    def d_head(self) -> int:
        return self.d_model // self.n_heads

    @property
    def vocab_padded(self) -> int:
        return -(-self.vocab // 64) * 64


class BlockSaved(NamedTuple):
    x: torch.Tensor
    rstd1: torch.Tensor
    h1: torch.Tensor
    qkv: torch.Tensor
    o: torch.Tensor
    lse: torch.Tensor
    x2: torch.Tensor
    rstd2: torch.Tensor
    h2: torch.Tensor
    gu: torch.Tensor
    hh: torch.Tensor


def block_forward(x, w: BlockWeights, cfg: EngineConfig, rope_cache, batch: int, seq: int, keep: bool, gather=None):
    """x (M, d) -> (y (M, d), saved activations or None).  ``gather`` is an optional pending all-gather
    (the next FSDP unit's weights) that the largest GEMM of the block carries."""
    h1, rstd1 = ops.rmsnorm_fwd(x, w.n1, cfg.eps)
    qkv = ops.gemm_qkv_rope(h1, w.wqkv, rope_cache, seq, cfg.n_heads)     # RoPE in the GEMM epilogue
    o, lse = ops.attention_fwd(qkv, batch, seq, cfg.n_heads)
    x2 = ops.gemm(o, w.wo, "nt", residual=x)
    h2, rstd2 = ops.rmsnorm_fwd(x2, w.n2, cfg.eps)
    gu, hh = ops.gemm_swiglu(h2, w.wgu, gather=gather)                    # SiLU(gate) * up in the GEMM epilogue
    y = ops.gemm(hh, w.wdown, "nt", residual=x2)
    saved = BlockSaved(x, rstd1, h1, qkv, o, lse, x2, rstd2, h2, gu, hh) if keep else None
    return y, saved


def block_backward(dy, w: BlockWeights, s: BlockSaved, gw: BlockWeights, cfg: EngineConfig, rope_cache,
                   batch: int, seq: int, gather=None, reduce=None):
    """Returns dx; writes every weight gradient of the block into the views in ``gw``.  ``gather`` (the
    previous unit's weights, needed next) rides on the first GEMM, ``reduce`` (the reduce-scatter of the unit
    whose backward has just finished) on the third."""
    # ---- feed-forward half
    dgu = ops.gemm_swiglu_bwd(dy, w.wdown, s.gu, gather=gather)          # SiLU*mul backward in the GEMM epilogue
    ops.gemm(dy, s.hh, "tn", out=gw.wdown)
    dh2 = ops.gemm(dgu, w.wgu, "nn", reduce=reduce)
    ops.gemm(dgu, s.h2, "tn", out=gw.wgu)
    del dgu
    dx2 = _norm_bwd(dh2, s.x2, w.n2, s.rstd2, gw.n2, dy)
    del dh2
    # ---- attention half
    do = ops.gemm(dx2, w.wo, "nn")
    ops.gemm(dx2, s.o, "tn", out=gw.wo)
    dqkv = ops.attention_bwd(do, s.qkv, s.o, s.lse, batch, seq, cfg.n_heads, rope_cache)   # dQ, dK rotated back
    del do
    dh1 = ops.gemm(dqkv, w.wqkv, "nn")
    ops.gemm(dqkv, s.h1, "tn", out=gw.wqkv)
    del dqkv
    dx = _norm_bwd(dh1, s.x, w.n1, s.rstd1, gw.n1, dx2)
    return dx


def _norm_bwd(dyn, x, w, rstd, dw_out, dres):
    """RMSNorm backward with the residual-branch gradient added in the same pass."""
    if dyn.is_cuda:
        from ..ops import native
        if dw_out.dtype == torch.float32:
            dx, _ = native.rmsnorm_bwd(dyn, x, w, rstd, dw_out=dw_out, dres=dres)
        else:
            dx, dw = native.rmsnorm_bwd(dyn, x, w, rstd, dres=dres)
            dw_out.copy_(dw)
        return dx
    dx, dw = ops.torch_impl.rmsnorm_bwd(dyn, x, w, rstd)
    dw_out.copy_(dw.to(dw_out.dtype))
    return dx + dres


def _seg_view(by_name, flat, name, base):
    seg = by_name[name]
    return flat[seg.start - base:seg.start - base + seg.numel].view(seg.shape)


def block_views(by_name, names: dict, flat: torch.Tensor, base: int) -> BlockWeights:
    """Views of one block's tensors inside ``flat``, whose element 0 is arena offset ``base``."""
    q = by_name[names["q"]]
    d = q.shape[1]
    wqkv = flat[q.start - base:q.start - base + 3 * q.numel].view(3 * q.shape[0], d)
    g = by_name[names["gate"]]
    if names.get("up") is None:           # merged (2F, d) parameter
        wgu = flat[g.start - base:g.start - base + g.numel].view(g.shape)
    else:
        wgu = flat[g.start - base:g.start - base + 2 * g.numel].view(2 * g.shape[0], d)
    return BlockWeights(wqkv, _seg_view(by_name, flat, names["o"], base), wgu,
                        _seg_view(by_name, flat, names["down"], base), _seg_view(by_name, flat, names["n1"], base),
                        _seg_view(by_name, flat, names["n2"], base))


def head_views(by_name, names: dict, flat: torch.Tensor, base: int) -> HeadWeights:
    """Embedding table, final norm and lm_head as views of ``flat`` (element 0 = arena offset ``base``)."""
    return HeadWeights(_seg_view(by_name, flat, names["emb"], base), _seg_view(by_name, flat, names["norm"], base),
                       _seg_view(by_name, flat, names["lm"], base))


class LocalProvider:
    """Weights and gradients taken from a model-local ``ParamArena``."""

    def __init__(self, arena, layer_names: list[dict], head_names: dict):
        self.arena = arena
        self.layer_names = layer_names
        self.head_names = head_names
        self.post_backward_hooks = []   # callables (kind, index) -> None; used by DDP
        self._w_cache = None
        self._g_cache = None
        self._cache_key = None

    def _views(self, flat):
        layers = [block_views(self.arena.by_name, names, flat, 0) for names in self.layer_names]
        return layers, head_views(self.arena.by_name, self.head_names, flat, 0)

    def begin_step(self):
        """Refresh the compute mirror (if stale) and the cached views."""
        flat = self.arena.mirror()
        key = (flat.data_ptr(), self.arena.grad.data_ptr() if self.arena.grad is not None else 0)
        if key != self._cache_key:
            self._w_cache = self._views(flat)
            self._g_cache = None
            self._cache_key = key

    def block_weights(self, i: int, backward: bool = False) -> BlockWeights:
        return self._w_cache[0][i]

    def head_weights(self, backward: bool = False) -> HeadWeights:
        return self._w_cache[1]

    def embed_weight(self) -> torch.Tensor:
        return self._w_cache[1].emb

    def embed_grad(self) -> torch.Tensor:
        return self._grads()[1].emb

    def _grads(self):
        if self._g_cache is None:
            self.arena.bind_grads()
            self._g_cache = self._views(self.arena.grad)
            self._cache_key = (self._cache_key[0], self.arena.grad.data_ptr())
        return self._g_cache

    def block_grads(self, i: int) -> BlockWeights:
        return self._grads()[0][i]

    def head_grads(self) -> HeadWeights:
        return self._grads()[1]

    def pre_backward(self, kind: str, i: int):
        pass

    def post_forward(self, kind: str, i: int):
        pass

    def take_gather(self, kind: str, i: int):
        return None

    def take_reduce(self, kind: str, i: int):
        return None

    def post_backward(self, kind: str, i: int):
        for h in self.post_backward_hooks:
            h(kind, i)
        if kind == "embed" and not self.arena.grads_bound:
            self.arena.bind_grads()


class _BlockFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, anchor, eng, i, batch, seq):
        w = eng.provider.block_weights(i)
        keep = torch.is_grad_enabled() or ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        cfg = eng.cfg
        with nvtx_range(f"block{i}.fwd"):
            y, saved = block_forward(x, w, cfg, eng.rope_cache, batch, seq, keep and not cfg.recompute,
                                     gather=eng.provider.take_gather("fwd", i))
        ctx.eng, ctx.i, ctx.batch, ctx.seq = eng, i, batch, seq
        ctx.saved = saved
        ctx.x_in = x if cfg.recompute else None
        eng.provider.post_forward("block", i)
        return y

    @staticmethod
    def backward(ctx, dy):
        eng, i = ctx.eng, ctx.i
        prov = eng.provider
        prov.pre_backward("block", i)
        w = prov.block_weights(i, backward=True)
        saved = ctx.saved
        if saved is None:
            with nvtx_range(f"block{i}.recompute"):
                _, saved = block_forward(ctx.x_in, w, eng.cfg, eng.rope_cache, ctx.batch, ctx.seq, True)
        with nvtx_range(f"block{i}.bwd"):
            dx = block_backward(dy.contiguous(), w, saved, prov.block_grads(i), eng.cfg, eng.rope_cache, ctx.batch,
                                ctx.seq, gather=prov.take_gather("bwd", i), reduce=prov.take_reduce("bwd", i))
        ctx.saved = None
        ctx.x_in = None
        prov.post_backward("block", i)
        return dx, None, None, None, None, None


class _EmbedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, anchor, eng):
        w = eng.provider.embed_weight()
        ctx.eng = eng
        ctx.tokens = tokens
        out = ops.embedding_fwd(tokens, w)
        eng.provider.post_forward("embed", 0)
        return out

    @staticmethod
    def backward(ctx, dx):
        prov = ctx.eng.provider
        prov.pre_backward("embed", 0)
        # fp32 gradient table, or the bf16 gradient staging of a multi-GPU run: each row is written once from the
        # fp32 sum of its token run, so no fp32 temporary of the table's size is needed
        ops.embedding_bwd(dx.contiguous(), ctx.tokens, prov.embed_grad())
        prov.post_backward("embed", 0)
        return None, None, None


class _HeadFn(torch.autograd.Function):
    """Final RMSNorm + lm_head producing materialised logits (API-compatible path)."""

    @staticmethod
    def forward(ctx, x, anchor, eng):
        hw = eng.provider.head_weights()
        cfg = eng.cfg
        hn, rstd = ops.rmsnorm_fwd(x, hw.norm, cfg.eps)
        buf = torch.empty((x.shape[0], cfg.vocab_padded), dtype=x.dtype, device=x.device)
        logits = buf[:, :cfg.vocab]
        ops.gemm(hn, hw.lm, "nt", out=logits, pad_writable=True)
        ctx.eng = eng
        ctx.saved = (x, rstd, hn)
        return logits

    @staticmethod
    def backward(ctx, dlogits):
        eng = ctx.eng
        prov = eng.provider
        prov.pre_backward("head", 0)
        hw = prov.head_weights(backward=True)
        gw = prov.head_grads()
        x, rstd, hn = ctx.saved
        ctx.saved = None
        if dlogits.stride(1) != 1 or dlogits.stride(0) % 8 != 0 or dlogits.data_ptr() % 16 != 0:
            buf = torch.zeros((dlogits.shape[0], eng.cfg.vocab_padded), dtype=x.dtype, device=x.device)
            buf[:, :eng.cfg.vocab] = dlogits
            dlogits = buf[:, :eng.cfg.vocab]
        elif dlogits.dtype != x.dtype:
            dlogits = dlogits.to(x.dtype)
        dhn = ops.gemm(dlogits, hw.lm, "nn")
        ops.gemm(dlogits, hn, "tn", out=gw.lm)
        dx = _head_norm_bwd(dhn, x, hw.norm, rstd, gw.norm)
        prov.post_backward("head", 0)
        return dx, None, None


def _head_norm_bwd(dyn, x, w, rstd, dw_out):
    if dyn.is_cuda:
        from ..ops import native
        if dw_out.dtype == torch.float32:
            dx, _ = native.rmsnorm_bwd(dyn, x, w, rstd, dw_out=dw_out)
        else:
            dx, dw = native.rmsnorm_bwd(dyn, x, w, rstd)
            dw_out.copy_(dw)
        return dx
    dx, dw = ops.torch_impl.rmsnorm_bwd(dyn, x, w, rstd)
    dw_out.copy_(dw.to(dw_out.dtype))
    return dx


class _HeadLossFn(torch.autograd.Function):
    """Final RMSNorm + lm_head + mean cross-entropy without ever holding the full logits.

    Rows are processed in chunks: logits chunk -> loss + d(logits) in place -> the chunk's
    contribution to d(hidden) and d(lm_head).  The gradients are produced during forward and
    scaled by the incoming gradient in backward, so one (chunk, V) buffer is all that is live.
    """

    @staticmethod
    def forward(ctx, x, anchor, eng, targets, chunk_rows):
        prov = eng.provider
        hw = prov.head_weights()
        cfg = eng.cfg
        m = x.shape[0]
        need_grad = torch.is_grad_enabled() or ctx.needs_input_grad[0]
        hn, rstd = ops.rmsnorm_fwd(x, hw.norm, cfg.eps)
        loss = torch.zeros((), dtype=torch.float32, device=x.device)
        n_valid = (targets != -100).sum().clamp(min=1).float()   # stays on the device
        buf = torch.empty((min(chunk_rows, m), cfg.vocab_padded), dtype=x.dtype, device=x.device)
        dhn = torch.empty_like(hn) if need_grad else None
        gw = prov.head_grads() if need_grad else None
        lm_acc = None
        for r0 in range(0, m, chunk_rows):
            r1 = min(m, r0 + chunk_rows)
            logits = buf[:r1 - r0, :cfg.vocab]
            ops.gemm(hn[r0:r1], hw.lm, "nt", out=logits, pad_writable=True)
            tg = targets[r0:r1]
            # every chunk is normalised by the global count of valid targets, so the parts simply add up
            if need_grad:
                ops.xent_fwd_bwd(buf[:r1 - r0], tg, 1.0, -100, cfg.vocab, loss_out=loss, accumulate_loss=(r0 > 0),
                                 n_valid=n_valid)
                ops.gemm(logits, hw.lm, "nn", out=dhn[r0:r1])
                if gw.lm.dtype == torch.float32:
                    ops.gemm(logits, hn[r0:r1], "tn", out=gw.lm, accumulate=(r0 > 0))
                else:
                    if lm_acc is None:
                        lm_acc = torch.empty(gw.lm.shape, dtype=torch.float32, device=x.device)
                    ops.gemm(logits, hn[r0:r1], "tn", out=lm_acc, accumulate=(r0 > 0))
            else:
                ops.xent_fwd(buf[:r1 - r0], tg, -100, cfg.vocab, loss_out=loss, accumulate_loss=(r0 > 0),
                             n_valid=n_valid)
        if need_grad and lm_acc is not None:
            gw.lm.copy_(lm_acc)
        ctx.eng = eng
        ctx.saved = (x, rstd, dhn)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        eng = ctx.eng
        prov = eng.provider
        prov.pre_backward("head", 0)
        hw = prov.head_weights(backward=True)
        gw = prov.head_grads()
        x, rstd, dhn = ctx.saved
        ctx.saved = None
        # The gradients were produced in forward for d(loss) = 1; apply the incoming factor on the
        # device (two bandwidth-bound launches, no host synchronisation).
        scale = dloss.to(torch.float32).reshape(())
        ops.scale_(dhn, scale)
        if gw.lm.is_contiguous() and gw.lm.dtype in (torch.float32, torch.bfloat16):
            ops.scale_(gw.lm, scale)
        else:
            gw.lm.mul_(scale.to(gw.lm.dtype))
        dx = _head_norm_bwd(dhn, x, hw.norm, rstd, gw.norm)
        prov.post_backward("head", 0)
        return dx, None, None, None, None


class NativeEngine:
    """Runs a ``TransformerLM``-shaped stack through the fused forward/backward."""

    def __init__(self, cfg: EngineConfig, provider, rope_cache: torch.Tensor):
        self.cfg = cfg
        self.provider = provider
        self.rope_cache = rope_cache
        # rows of logits that exist at a time in the fused head + loss (B200_LOSS_CHUNK_ROWS overrides)
        self.loss_chunk_rows = int(os.environ.get("B200_LOSS_CHUNK_ROWS", "4096"))

    def _anchor(self):
        return self.provider.arena.anchor

    def hidden(self, tokens: torch.Tensor) -> tuple[torch.Tensor, int, int]:
        seq = tokens.shape[-1]
        batch = tokens.numel() // seq
        self.provider.begin_step()
        anchor = self._anchor()
        flat = tokens.reshape(-1).contiguous()
        x = _EmbedFn.apply(flat, anchor, self)
        for i in range(self.cfg.n_layers):
            x = _BlockFn.apply(x, anchor, self, i, batch, seq)
        return x, batch, seq

    def logits(self, tokens: torch.Tensor) -> torch.Tensor:
        x, batch, seq = self.hidden(tokens)
        out = _HeadFn.apply(x, self._anchor(), self)
        return out.view(*tokens.shape, self.cfg.vocab) if out.is_contiguous() else out.unflatten(0, tuple(tokens.shape))

    def loss(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        x, batch, seq = self.hidden(tokens)
        return _HeadLossFn.apply(x, self._anchor(), self, targets.reshape(-1).contiguous(), self.loss_chunk_rows)
