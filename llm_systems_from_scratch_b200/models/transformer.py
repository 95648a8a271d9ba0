"""Decoder-only Transformer language model (RMSNorm, interleaved RoPE, SwiGLU, causal MHA).

Public surface and state-dict layout follow the reference model
(llm-core/llm_core/model.py:21-393): ``TransformerLM(vocab_size, context_length, d_model,
num_layers, num_heads, d_ff, rope_theta, use_flash_attn=False, use_custom_triton=False)`` with
``.token_embeddings / .positional_encoder / .layers / .final_norm / .lm_head``, an untied output
head, ``forward -> logits``, ``generate``, ``from_pretrained`` and ``get_num_params``.

Two execution paths share the same parameters:

* eager  - plain PyTorch modules, any device/dtype; the numerical oracle.
* native - selected by ``use_custom_triton=True`` (the reference's "custom kernel" switch).  The
  whole stack then runs through ``models.engine.NativeEngine``: parameters live in one flat arena,
  each block is a single autograd node built from fused sm_100a kernels, compute is bf16 with fp32
  accumulation and fp32 master weights.  On CPU the same engine runs on the fp32 PyTorch statements
  of those kernels, which is how its hand-written backward is tested without a GPU.

Fixes relative to the reference, kept behind the same signatures: ``top_k`` really filters
(model.py:225 discards its result), ``temperature == 0`` means greedy decoding, and checkpoints
written with either FFN key layout (split gate/up or merged ``w_gate_up``) load into either model.
"""
from __future__ import annotations

import json
import logging
import math

import torch
from torch import Tensor, nn

from ..ops import functional as Fn
from .arena import ParamArena
from .engine import EngineConfig, LocalProvider, NativeEngine

logger = logging.getLogger(__name__)


def _trunc_normal(shape, std: float) -> Tensor:
    t = torch.empty(*shape)
    nn.init.trunc_normal_(t, mean=0.0, std=std, a=-3.0 * std, b=3.0 * std)
    return t


class Linear(nn.Module):
    """Bias-free affine map; weight is (d_out, d_in), init N(0, 2/(d_in+d_out)) truncated at 3 sigma."""

    def __init__(self, d_in: int, d_out: int):
        super().__init__()
        self.weight = nn.Parameter(_trunc_normal((d_out, d_in), math.sqrt(2.0 / (d_in + d_out))))

    def forward(self, x: Tensor) -> Tensor:
        return torch.nn.functional.linear(x, self.weight)

    def extra_repr(self) -> str:
        return f"d_in={self.weight.shape[1]}, d_out={self.weight.shape[0]}"


class Embedding(nn.Module):
    """Token lookup table (vocab, d_model), init N(0, 1) truncated at +-3."""

    def __init__(self, vocab_size: int, d_model: int):
        super().__init__()
        self.weight = nn.Parameter(_trunc_normal((vocab_size, d_model), 1.0))

    def forward(self, token_ids: Tensor) -> Tensor:
        return torch.nn.functional.embedding(token_ids, self.weight)

    def extra_repr(self) -> str:
        return f"vocab_size={self.weight.shape[0]}, d_model={self.weight.shape[1]}"


class RMSNorm(nn.Module):
    """y = x / sqrt(mean(x^2) + eps) * weight, computed in fp32 and cast back."""

    def __init__(self, d_model: int, eps: float = 1e-5, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d_model, device=device))
        self.eps = eps

    def forward(self, x: Tensor) -> Tensor:
        xf = x.float()
        inv = torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + self.eps)
        return (self.weight * (xf * inv)).to(x.dtype)

    def extra_repr(self) -> str:
        return f"d_model={self.weight.shape[0]}, eps={self.eps}"


class RotaryEmbedding(nn.Module):
    """Rotary position encoding over adjacent pairs (x[2i], x[2i+1]).

    ``_freq_cache`` is a non-persistent buffer (2, context_length, d/2) holding cos and sin of
    ``pos * theta^(-2i/d)``; one instance is shared by every layer.
    """

    def __init__(self, context_length: int, d: int, theta: float = 10000.0):
        super().__init__()
        self.register_buffer("_freq_cache", self._build_cache(context_length, d, theta), persistent=False)

    @staticmethod
    def _build_cache(context_length: int, d: int, theta: float) -> Tensor:
        if d % 2:
            raise ValueError("rotary dimension must be even")
        inv_freq = theta ** -(torch.arange(0, d, 2) / d)
        angles = torch.outer(torch.arange(context_length).float(), inv_freq)
        return torch.stack((angles.cos(), angles.sin()))

    def forward(self, x: Tensor, pos_ids: Tensor) -> Tensor:
        cos, sin = self._freq_cache[:, pos_ids, :]
        pairs = x.unflatten(-1, (-1, 2))
        even, odd = pairs[..., 0], pairs[..., 1]
        rotated = torch.stack((cos * even - sin * odd, sin * even + cos * odd), dim=-1)
        return rotated.flatten(-2)

    def extra_repr(self) -> str:
        return f"context_length={self._freq_cache.shape[1]}, d={self._freq_cache.shape[2] * 2}"


def silu(x: Tensor) -> Tensor:
    return x * torch.sigmoid(x)


class SwiGLU(nn.Module):
    """down(silu(gate(x)) * up(x)) with three separate projections."""

    def __init__(self, d_model: int, d_ff: int):
        super().__init__()
        self.gate_proj = Linear(d_model, d_ff)
        self.down_proj = Linear(d_ff, d_model)
        self.up_proj = Linear(d_model, d_ff)

    def forward(self, x: Tensor) -> Tensor:
        return self.down_proj(silu(self.gate_proj(x)) * self.up_proj(x))


class FusedSwiGLU(nn.Module):
    """SwiGLU with gate and up merged into one (2*d_ff, d_model) projection, gate rows first.

    Same parameter names as the reference's fused module
    (llm-systems/llm_systems/kernels/triton_swiglu.py:161-197): ``w_gate_up`` and ``w_down``.
    """

    def __init__(self, d_model: int, d_ff: int):
        super().__init__()
        self.d_ff = d_ff
        self.w_gate_up = Linear(d_model, 2 * d_ff)
        self.w_down = Linear(d_ff, d_model)
        with torch.no_grad():  # each half initialised like an independent (d_ff, d_model) Linear
            std = math.sqrt(2.0 / (d_model + d_ff))
            self.w_gate_up.weight.copy_(_trunc_normal((2 * d_ff, d_model), std))

    def forward(self, x: Tensor) -> Tensor:
        gate, up = self.w_gate_up(x).split(self.d_ff, dim=-1)
        return self.w_down(silu(gate) * up)


def scaled_dot_product_attention(Q: Tensor, K: Tensor, V: Tensor, mask: Tensor | None = None) -> Tensor:
    """softmax(Q K^T / sqrt(d_k) [masked]) V; ``mask`` is True where attention is allowed."""
    scores = Q @ K.transpose(-1, -2) / math.sqrt(K.shape[-1])
    if mask is not None:
        scores = scores.masked_fill(~mask, float("-inf"))
    return Fn.softmax(scores, dim=-1) @ V


class CausalMultiHeadSelfAttention(nn.Module):
    def __init__(self, d_model: int, num_heads: int, positional_encoder: RotaryEmbedding,
                 use_flash_attn: bool = False):
        super().__init__()
        if d_model % num_heads:
            raise ValueError("d_model must be divisible by num_heads")
        self.d_model, self.num_heads, self.use_flash_attn = d_model, num_heads, use_flash_attn
        self.d_head = d_model // num_heads
        self.q_proj = Linear(d_model, d_model)
        self.k_proj = Linear(d_model, d_model)
        self.v_proj = Linear(d_model, d_model)
        self.output_proj = Linear(d_model, d_model)
        self.positional_encoder = positional_encoder

    def _heads(self, t: Tensor) -> Tensor:
        return t.unflatten(-1, (self.num_heads, self.d_head)).transpose(-2, -3)

    def forward(self, x: Tensor, token_positions: Tensor | None = None) -> Tensor:
        seq = x.shape[-2]
        q, k, v = self._heads(self.q_proj(x)), self._heads(self.k_proj(x)), self._heads(self.v_proj(x))
        if token_positions is None:
            token_positions = torch.arange(seq, device=x.device)
        pos = token_positions.unsqueeze(-2) if token_positions.dim() > 1 else token_positions
        q, k = self.positional_encoder(q, pos), self.positional_encoder(k, pos)
        if self.use_flash_attn:
            q, k = q.to(v.dtype), k.to(v.dtype)
            out = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
        else:
            allowed = torch.ones(seq, seq, dtype=torch.bool, device=x.device).tril()
            out = scaled_dot_product_attention(q, k, v, allowed)
        return self.output_proj(out.transpose(-2, -3).flatten(-2))


class TransformerBlock(nn.Module):
    """x + attn(norm(x)), then x + ffn(norm(x))."""

    def __init__(self, d_model: int, num_heads: int, d_ff: int, positional_encoder: RotaryEmbedding,
                 use_flash_attn: bool = False, use_custom_triton: bool = False):
        super().__init__()
        self.attn = CausalMultiHeadSelfAttention(d_model, num_heads, positional_encoder, use_flash_attn)
        self.ffn = FusedSwiGLU(d_model, d_ff) if use_custom_triton else SwiGLU(d_model, d_ff)
        self.attn_norm = RMSNorm(d_model)
        self.ffn_norm = RMSNorm(d_model)

    def forward(self, x: Tensor) -> Tensor:
        x = x + self.attn(self.attn_norm(x))
        return x + self.ffn(self.ffn_norm(x))


class TransformerLM(nn.Module):
    def __init__(self, vocab_size: int, context_length: int, d_model: int, num_layers: int, num_heads: int,
                 d_ff: int, rope_theta: float, use_flash_attn: bool = False, use_custom_triton: bool = False):
        self.config = dict(vocab_size=vocab_size, context_length=context_length, d_model=d_model,
                           num_layers=num_layers, num_heads=num_heads, d_ff=d_ff, rope_theta=rope_theta,
                           use_flash_attn=use_flash_attn, use_custom_triton=use_custom_triton)
        super().__init__()
        self.vocab_size, self.context_length, self.d_model = vocab_size, context_length, d_model
        self.num_heads, self.d_ff, self.num_layers = num_heads, d_ff, num_layers
        self.use_custom_triton = use_custom_triton
        self.token_embeddings = Embedding(vocab_size, d_model)
        self.positional_encoder = RotaryEmbedding(context_length, d_model // num_heads, rope_theta)
        self.layers = nn.ModuleList(
            TransformerBlock(d_model, num_heads, d_ff, self.positional_encoder, use_flash_attn, use_custom_triton)
            for _ in range(num_layers))
        self.final_norm = RMSNorm(d_model)
        self.lm_head = Linear(d_model, vocab_size)
        self._engine: NativeEngine | None = None
        self.activation_checkpointing = False
        self._register_load_state_dict_pre_hook(self._convert_ffn_keys)
        logger.info(f"non-embedding parameters: {self.get_num_params() / 1e6:.2f}M")

    # ------------------------------------------------------------------ bookkeeping
    def get_num_params(self, non_embedding: bool = True) -> int:
        n = sum(p.numel() for p in self.parameters())
        return n - self.lm_head.weight.numel() if non_embedding else n

    def _convert_ffn_keys(self, state_dict, prefix, *args):
        """Accept checkpoints in either FFN layout (split gate/up/down or merged w_gate_up/w_down)."""
        for i, layer in enumerate(self.layers):
            base = f"{prefix}layers.{i}.ffn."
            merged = isinstance(layer.ffn, FusedSwiGLU)
            if merged and base + "gate_proj.weight" in state_dict:
                gate = state_dict.pop(base + "gate_proj.weight")
                up = state_dict.pop(base + "up_proj.weight")
                state_dict[base + "w_gate_up.weight"] = torch.cat((gate, up), dim=0)
                state_dict[base + "w_down.weight"] = state_dict.pop(base + "down_proj.weight")
            elif not merged and base + "w_gate_up.weight" in state_dict:
                gate, up = state_dict.pop(base + "w_gate_up.weight").chunk(2, dim=0)
                state_dict[base + "gate_proj.weight"] = gate
                state_dict[base + "up_proj.weight"] = up
                state_dict[base + "down_proj.weight"] = state_dict.pop(base + "w_down.weight")

    def canonical_state_dict(self) -> dict:
        """State dict with split FFN keys (the layout every reference model without the fused
        module expects), independent of which FFN module this instance holds."""
        out = {}
        for k, v in self.state_dict().items():
            if k.endswith("ffn.w_gate_up.weight"):
                gate, up = v.chunk(2, dim=0)
                out[k.replace("w_gate_up", "gate_proj")] = gate
                out[k.replace("w_gate_up", "up_proj")] = up
            elif k.endswith("ffn.w_down.weight"):
                out[k.replace("w_down", "down_proj")] = v
            else:
                out[k] = v
        return out

    # ---------------------------------------------------------------- native engine
    def native_supported(self) -> bool:
        dh = self.d_model // self.num_heads
        ok = self.use_custom_triton and self.d_model % 8 == 0 and self.d_ff % 8 == 0 and dh % 8 == 0
        if ok and next(self.parameters()).is_cuda:
            ok = dh in (32, 64, 128)
        return bool(ok)

    def _apply(self, fn, *args, **kwargs):
        # .to()/.cuda()/.float() re-create parameter storage: the arena must be rebuilt afterwards.
        self._engine = None
        for p in self.parameters():
            if hasattr(p, "_arena"):
                del p._arena
        return super()._apply(fn, *args, **kwargs)

    def engine(self) -> NativeEngine:
        """Build (once per placement) the flat parameter arena and the fused execution engine."""
        if self._engine is not None:
            return self._engine
        ordered, groups, layer_names = [], [], []
        for i, layer in enumerate(self.layers):
            first = len(ordered)
            pre = f"layers.{i}."
            names = {"q": pre + "attn.q_proj.weight", "o": pre + "attn.output_proj.weight",
                     "n1": pre + "attn_norm.weight", "n2": pre + "ffn_norm.weight"}
            ordered += [(names["q"], layer.attn.q_proj.weight), (pre + "attn.k_proj.weight", layer.attn.k_proj.weight),
                        (pre + "attn.v_proj.weight", layer.attn.v_proj.weight), (names["o"], layer.attn.output_proj.weight)]
            if isinstance(layer.ffn, FusedSwiGLU):
                names.update(gate=pre + "ffn.w_gate_up.weight", up=None, down=pre + "ffn.w_down.weight")
                ordered += [(names["gate"], layer.ffn.w_gate_up.weight), (names["down"], layer.ffn.w_down.weight)]
            else:
                names.update(gate=pre + "ffn.gate_proj.weight", up=pre + "ffn.up_proj.weight",
                             down=pre + "ffn.down_proj.weight")
                ordered += [(names["gate"], layer.ffn.gate_proj.weight), (names["up"], layer.ffn.up_proj.weight),
                            (names["down"], layer.ffn.down_proj.weight)]
            ordered += [(names["n1"], layer.attn_norm.weight), (names["n2"], layer.ffn_norm.weight)]
            groups.append((f"layer{i}", first, len(ordered) - 1))
            layer_names.append(names)
        first = len(ordered)
        head_names = {"emb": "token_embeddings.weight", "norm": "final_norm.weight", "lm": "lm_head.weight"}
        ordered += [(head_names["emb"], self.token_embeddings.weight), (head_names["norm"], self.final_norm.weight),
                    (head_names["lm"], self.lm_head.weight)]
        groups.append(("head", first, len(ordered) - 1))
        groups.append(("embed", first, first))                     # FSDP shards the table and the head separately
        groups.append(("lmhead", first + 1, len(ordered) - 1))
        dev = ordered[0][1].device
        if any(p.device != dev or p.dtype != torch.float32 for _, p in ordered):
            raise RuntimeError("the native engine needs all parameters in fp32 on one device")
        seg_align = ParamArena.ALIGN
        if (self.d_model * self.d_model) % seg_align or (self.d_ff * self.d_model) % seg_align:
            raise RuntimeError("d_model*d_model and d_ff*d_model must be multiples of 64 for the fused QKV / gate-up views")
        arena = ParamArena(ordered, groups)
        cfg = EngineConfig(self.d_model, self.num_heads, self.d_ff, self.vocab_size, self.num_layers,
                           eps=self.final_norm.eps, recompute=self.activation_checkpointing)
        provider = LocalProvider(arena, layer_names, head_names)
        rope = self.positional_encoder._freq_cache.to(device=dev, dtype=torch.float32).contiguous()
        self._engine = NativeEngine(cfg, provider, rope)
        return self._engine

    def zero_grad(self, set_to_none: bool = True):
        eng = self._engine
        if eng is not None and eng.provider.arena.grads_bound:
            return  # every gradient slice is fully overwritten by the next backward
        super().zero_grad(set_to_none=set_to_none)

    # ---------------------------------------------------------------------- forward
    def forward(self, token_ids: Tensor) -> Tensor:
        if self.native_supported():
            return self.engine().logits(token_ids)
        x = self.token_embeddings(token_ids)
        for layer in self.layers:
            x = layer(x)
        return self.lm_head(self.final_norm(x))

    def loss(self, token_ids: Tensor, targets: Tensor) -> Tensor:
        """Mean next-token cross-entropy.  On the native path the logits are never materialised."""
        if self.native_supported():
            return self.engine().loss(token_ids, targets)
        logits = self.forward(token_ids)
        return Fn.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1))

    # ------------------------------------------------------------------- generation
    @torch.no_grad()
    def generate(self, prompt_ids: Tensor, max_new_tokens: int, temperature: float = 1.0,
                 top_k: int | None = None, eos_token_id: int | None = None) -> Tensor:
        """Sample up to ``max_new_tokens`` continuation ids; returns only the new ids, shape (1, n).

        With the fused engine a single prompt that fits the context window runs through the paged-KV serving engine
        (one prefill, then one cached decode step per token) instead of re-running the whole context for every
        token as the reference does (llm-core/llm_core/model.py:210-233); longer generations slide the window with
        the re-forward loop below, which is also what the eager model uses."""
        ids = prompt_ids.unsqueeze(0) if prompt_ids.dim() == 1 else prompt_ids
        if (self.native_supported() and ids.shape[0] == 1 and max_new_tokens > 0
                and 0 < ids.shape[1] and ids.shape[1] + max_new_tokens <= self.context_length):
            from ..serving import ServingEngine
            need = -(-(ids.shape[1] + max_new_tokens) // 16) + 1
            eng = ServingEngine(self, num_pages=need, page_size=16, max_batch=1, use_cuda_graphs=False)
            out = eng.generate([ids[0].tolist()], max_new_tokens, eos_token_id, temperature, top_k)[0]
            if eos_token_id is not None and out and out[-1] == eos_token_id:
                out = out[:-1]                       # the contract of this method: the stop token is not returned
            return torch.tensor([out], dtype=torch.long, device=ids.device).reshape(1, -1)
        new: list[Tensor] = []
        for _ in range(max_new_tokens):
            window = ids[:, -self.context_length:]
            logits = self.forward(window)[:, -1]
            if logits.is_cuda and logits.dtype == torch.bfloat16 and temperature != 0:
                # filter, softmax and draw in one kernel (no sort, no probabilities in memory)
                from ..ops import native
                u = torch.rand(logits.shape[0], device=logits.device)
                nxt = native.sample_topk(logits.contiguous(), u, temperature, top_k).unsqueeze(-1)
                if eos_token_id is not None and int(nxt) == eos_token_id:
                    break
                ids = torch.cat((ids, nxt), dim=-1)
                new.append(nxt)
                continue
            last = logits.float()
            if temperature == 0:
                nxt = last.argmax(dim=-1, keepdim=True)
            else:
                last = last / temperature
                if top_k:
                    kth = torch.topk(last, min(top_k, last.shape[-1])).values[:, -1:]
                    last = last.masked_fill(last < kth, float("-inf"))
                nxt = torch.multinomial(Fn.softmax(last, dim=-1), 1)
            if eos_token_id is not None and int(nxt) == eos_token_id:
                break
            ids = torch.cat((ids, nxt), dim=-1)
            new.append(nxt)
        return torch.cat(new, dim=-1) if new else ids[:, :0]

    @classmethod
    def from_pretrained(cls, config_path: str, checkpoint_path: str) -> "TransformerLM":
        with open(config_path) as f:
            model = cls(**json.load(f))
        state = torch.load(checkpoint_path, map_location="cpu")
        state = state.get("model", state) if isinstance(state, dict) else state
        state = {(k[len("_orig_mod."):] if k.startswith("_orig_mod.") else k): v for k, v in state.items()}
        model.load_state_dict(state)
        return model
