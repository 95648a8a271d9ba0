"""CPU unit tests: functional ops, schedule, optimizer order, loader, tokenizer, checkpoints, watchdog."""
import ctypes
import json
import math
import os
import time

import numpy as np
import pytest
import torch

from llm_systems_from_scratch_b200.models.transformer import (Linear, RMSNorm, RotaryEmbedding, TransformerLM,
                                                               scaled_dot_product_attention)
from llm_systems_from_scratch_b200.ops import functional as Fn
from llm_systems_from_scratch_b200.optim import AdamW, FusedAdamW, cosine_lr_schedule

DATA = os.path.join(os.path.dirname(__file__), "data")
TINY = dict(vocab_size=97, context_length=16, d_model=32, num_layers=2, num_heads=4, d_ff=64, rope_theta=10000.0)


def test_softmax_family_and_loss():
    x = torch.randn(5, 11) * 30
    assert torch.allclose(Fn.softmax(x), torch.softmax(x, -1), atol=1e-6)
    assert torch.allclose(Fn.log_softmax(x), torch.log_softmax(x, -1), atol=1e-5)
    t = torch.randint(0, 11, (5,))
    assert torch.allclose(Fn.cross_entropy(x, t), torch.nn.functional.cross_entropy(x, t), atol=1e-5)


def test_clip_gradient_global_norm():
    ps = [torch.nn.Parameter(torch.randn(7, 3)), torch.nn.Parameter(torch.randn(5))]
    for p in ps:
        p.grad = torch.randn_like(p) * 10
    norm = math.sqrt(sum(float((p.grad ** 2).sum()) for p in ps))
    Fn.clip_gradient(ps, 1.0)
    new = math.sqrt(sum(float((p.grad ** 2).sum()) for p in ps))
    assert abs(new - 1.0 / (1 + 1e-6 / norm)) < 1e-4
    before = [p.grad.clone() for p in ps]
    Fn.clip_gradient(ps, 100.0)      # below the threshold: untouched
    assert all(torch.equal(a, p.grad) for a, p in zip(before, ps))


def test_cosine_schedule_edges():
    f = lambda s: cosine_lr_schedule(s, 1.0, 0.1, 10, 110)
    assert f(0) == 0.0 and abs(f(5) - 0.5) < 1e-12 and abs(f(10) - 1.0) < 1e-12
    assert abs(f(60) - 0.55) < 1e-12 and abs(f(110) - 0.1) < 1e-12 and f(500) == 0.1
    assert cosine_lr_schedule(0, 1.0, 0.1, 0, 10) == 1.0


def test_adamw_decay_applied_after_update():
    p = torch.nn.Parameter(torch.tensor([1.0, -2.0]))
    p.grad = torch.tensor([0.5, 0.25])
    opt = AdamW([p], lr=0.1, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.5)
    opt.step()
    m = 0.1 * p.grad
    v = 0.05 * p.grad ** 2
    alpha = 0.1 * math.sqrt(1 - 0.95) / (1 - 0.9)
    expect = torch.tensor([1.0, -2.0]) - alpha * m / (v.sqrt() + 1e-8)
    expect = expect - 0.1 * 0.5 * expect
    assert torch.allclose(p.data, expect, atol=1e-6)
    assert opt.state[p]["t"] == 2
    q = torch.nn.Parameter(torch.tensor([1.0, -2.0]))
    q.grad = torch.tensor([0.5, 0.25])
    FusedAdamW([q], lr=0.1, weight_decay=0.5).step()
    assert torch.allclose(q.data, expect, atol=1e-6)


def test_init_and_modules():
    torch.manual_seed(0)
    lin = Linear(64, 256)
    std = math.sqrt(2 / (64 + 256))
    assert lin.weight.shape == (256, 64) and lin.weight.abs().max() <= 3 * std + 1e-6
    assert abs(lin.weight.std().item() - std) < 0.1 * std
    x = torch.randn(3, 5, 64)
    n = RMSNorm(64)
    ref = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5)
    assert torch.allclose(n(x), ref, atol=1e-5)
    rope = RotaryEmbedding(32, 8, 10000.0)
    assert rope._freq_cache.shape == (2, 32, 4) and "_freq_cache" not in rope.state_dict()
    v = torch.randn(2, 4, 6, 8)
    r = rope(v, torch.arange(6))
    assert torch.allclose(r[..., 0, :], v[..., 0, :], atol=1e-6)           # position 0 is the identity
    assert torch.allclose(r.norm(dim=-1), v.norm(dim=-1), atol=1e-5)        # rotations preserve norms
    ang = 3 * 10000.0 ** (-2 / 8)
    e, o = v[0, 0, 3, 2], v[0, 0, 3, 3]
    assert abs(r[0, 0, 3, 2] - (math.cos(ang) * e - math.sin(ang) * o)) < 1e-5
    q = torch.randn(2, 3, 5, 8)
    mask = torch.ones(5, 5, dtype=torch.bool).tril()
    a = scaled_dot_product_attention(q, q, q, mask)
    b = torch.nn.functional.scaled_dot_product_attention(q, q, q, is_causal=True)
    assert torch.allclose(a, b, atol=1e-5)


def test_state_dict_keys_match_reference_layout():
    m = TransformerLM(**TINY)
    keys = list(m.state_dict().keys())
    assert keys[0] == "token_embeddings.weight" and keys[-2:] == ["final_norm.weight", "lm_head.weight"]
    per_layer = ["attn.q_proj.weight", "attn.k_proj.weight", "attn.v_proj.weight", "attn.output_proj.weight",
                 "ffn.gate_proj.weight", "ffn.down_proj.weight", "ffn.up_proj.weight", "attn_norm.weight",
                 "ffn_norm.weight"]
    assert keys[1:10] == [f"layers.0.{k}" for k in per_layer]
    assert len(keys) == 3 + 9 * TINY["num_layers"]
    assert set(m.config) == {"vocab_size", "context_length", "d_model", "num_layers", "num_heads", "d_ff", "rope_theta",
                             "use_flash_attn", "use_custom_triton"}
    assert m.get_num_params() == sum(p.numel() for p in m.parameters()) - m.lm_head.weight.numel()
    fused = TransformerLM(**TINY, use_custom_triton=True)
    assert "layers.0.ffn.w_gate_up.weight" in fused.state_dict() and fused.state_dict()["layers.0.ffn.w_gate_up.weight"].shape == (128, 32)


def test_sample_batch_and_sampler():
    from llm_systems_from_scratch_b200.data import BatchSampler, sample_batch
    tokens = np.arange(1000, dtype=np.uint32)
    x, y = sample_batch(tokens, 4, 16, "cpu")
    assert x.dtype == torch.int64 and x.shape == (4, 16) and torch.equal(x + 1, y)
    a = BatchSampler(tokens, 4, 16, "cpu", seed=3, rank=1)
    b = BatchSampler(tokens, 4, 16, "cpu", seed=3, rank=1)
    c = BatchSampler(tokens, 4, 16, "cpu", seed=3, rank=2)
    xa, _ = a.next()
    xb, _ = b.next()
    xc, _ = c.next()
    assert torch.equal(xa, xb) and not torch.equal(xa, xc)


def test_tokenizer_matches_reference_golden_files(tmp_path):
    from llm_systems_from_scratch_b200.tokenizer import BPETokenizer, Tokenizer
    ref = Tokenizer.from_files(os.path.join(DATA, "vocab.json"), os.path.join(DATA, "merges.json"), ["<|endoftext|>"])
    tr = BPETokenizer()
    vocab, merges = tr.train(os.path.join(DATA, "corpus.txt"), len(ref.id_to_bytes), ["<|endoftext|>"], verbose=False)
    assert merges == ref.merges and vocab == ref.id_to_bytes          # same merges, same order, same ids
    assert vocab[0] == b"<|endoftext|>" and vocab[1] == b"\x00" and vocab[256] == b"\xff"
    tr.save(tmp_path / "v.json", tmp_path / "m.json")
    again = Tokenizer.from_files(tmp_path / "v.json", tmp_path / "m.json", ["<|endoftext|>"])
    text = open(os.path.join(DATA, "corpus.txt"), encoding="utf-8").read()
    ids = again.encode(text)
    assert ids == np.fromfile(os.path.join(DATA, "corpus.bin"), dtype=np.uint32).tolist()
    assert again.decode(ids) == text
    odd = "naïve café 🙂<|endoftext|>tail"
    enc = again.encode(odd)
    assert 0 in enc and again.decode(enc) == odd
    assert list(again.encode_iterable(["ab", "cd"])) == again.encode("ab") + again.encode("cd")
    extra = Tokenizer(vocab, merges, ["<|pad|>"])
    assert extra.encode("<|pad|>") == [len(vocab)]


def test_checkpoint_roundtrip_and_from_pretrained(tmp_path):
    from llm_systems_from_scratch_b200.utils.checkpoint import load_checkpoint, save_checkpoint
    torch.manual_seed(0)
    m = TransformerLM(**TINY)
    opt = AdamW(m.parameters(), lr=1e-2)
    x = torch.randint(0, 97, (2, 16))
    m.loss(x, x).backward()
    opt.step()
    path = str(tmp_path / "run" / "ckpt_3.pt")
    save_checkpoint(m, opt, 3, path)
    raw = torch.load(path)
    assert set(raw) == {"model", "iteration", "optimizer"} and raw["iteration"] == 3
    assert set(raw["optimizer"]["state"][0]) == {"t", "m", "v"}
    cfg = json.load(open(tmp_path / "run" / "model_config.json"))
    assert cfg == m.config
    m2 = TransformerLM(**TINY)
    opt2 = AdamW(m2.parameters(), lr=1e-2)
    assert load_checkpoint(path, m2, opt2) == 3
    assert all(torch.equal(a, b) for a, b in zip(m.state_dict().values(), m2.state_dict().values()))
    m3 = TransformerLM.from_pretrained(str(tmp_path / "run" / "model_config.json"), path)
    assert torch.equal(m3.lm_head.weight, m.lm_head.weight)
    # a fused-FFN model loads the split-key checkpoint
    m4 = TransformerLM(**TINY, use_custom_triton=True)
    m4.load_state_dict(raw["model"])
    assert torch.allclose(m4(x).float(), m(x), atol=1e-4)


def test_heartbeat_detects_silent_rank_and_step_watchdog():
    from llm_systems_from_scratch_b200.utils.watchdog import Heartbeat, RankFailure, StepWatchdog

    class Store(dict):
        def set(self, k, v):
            self[k] = v.encode()

        def get(self, k):
            return self[k]

    s = Store()
    a = Heartbeat(s, 0, 2, interval=0.05, timeout=0.3).start()
    b = Heartbeat(s, 1, 2, interval=0.05, timeout=0.3).start()
    time.sleep(0.2)
    a.check()
    b.pause()                     # host-side fault injection: rank 1 stops beating
    time.sleep(0.5)
    with pytest.raises(RankFailure) as e:
        a.check()
    assert e.value.dead == [1]
    b.mark_done()                 # a rank that finished is not a failure
    a.check()
    a.stop(), b.stop()
    w = StepWatchdog(0.1)
    w.arm()
    time.sleep(0.4)
    assert w.expired
    w.stop()


def test_fused_op_front_ends_on_cpu():
    """The fused front ends fall back to their fp32 statements on CPU tensors."""
    import torch
    from llm_systems_from_scratch_b200 import ops
    torch.manual_seed(0)
    m, d, f = 12, 16, 24
    dy, w2, gu = torch.randn(m, d), torch.randn(d, f), torch.randn(m, 2 * f)
    got = ops.gemm_swiglu_bwd(dy, w2, gu)
    dh = dy @ w2
    g, u = gu[:, :f], gu[:, f:]
    s = torch.sigmoid(g)
    want = torch.cat([dh * u * (s + g * s * (1 - s)), dh * g * s], dim=1)
    assert torch.allclose(got, want, atol=1e-5)
    x, wgu = torch.randn(m, d), torch.randn(2 * f, d)
    gu2, h = ops.gemm_swiglu(x, wgu)
    assert torch.allclose(gu2, x @ wgu.t(), atol=1e-5)
    assert torch.allclose(h, torch.nn.functional.silu(gu2[:, :f]) * gu2[:, f:], atol=1e-5)


def test_sample_topk_statement():
    """Inverse-CDF top-k sampling: support is the top-k set and frequencies follow the softmax."""
    import torch
    from llm_systems_from_scratch_b200 import ops
    torch.manual_seed(1)
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 3.0, 0.5, -2.0, 1.5]])
    n = 20000
    draws = ops.sample_topk(logits.expand(n, 8), torch.rand(n), 0.8, 5)
    freq = torch.bincount(draws, minlength=8).float() / n
    x = logits[0] / 0.8
    keep = x >= torch.topk(x, 5).values[-1]
    p = torch.softmax(x.masked_fill(~keep, float("-inf")), dim=0)
    assert freq[~keep].sum().item() == 0
    assert (freq - p).abs().max().item() < 0.015
    assert torch.equal(ops.sample_topk(logits, torch.tensor([0.3]), 1.0, 1), torch.tensor([4]))


def test_split_k_plan_for_decode_shapes():
    """The launcher's choice of tile width and K slices is host arithmetic: long contractions at decode sizes are
    split, a problem with more tiles than SMs is not, and every plan fits the scratch the Python side allocates."""
    from llm_systems_from_scratch_b200.ops import native
    if native.load(required=False) is None:
        pytest.skip("kernel library not built")
    lib = native.load()
    lib.b200_gemm_splitk_ws_floats.restype = ctypes.c_longlong
    ws_floats, counters = lib.b200_gemm_splitk_ws_floats(), lib.b200_gemm_splitk_counters()
    for m in (1, 64, 128, 256):
        for n, k in ((6144, 2048), (2048, 2048), (11008, 2048), (2048, 5504), (50264, 2048), (1000, 320)):
            bn, s = native.splitk_plan(m, n, k)
            assert bn in (64, 128, 256) and 1 <= s <= 8
            tiles = -(-m // 128) * -(-n // bn)
            assert s == 1 or (tiles * s * 128 * bn <= ws_floats and tiles * 4 <= counters and s <= (k + 63) // 64)
    assert native.splitk_plan(128, 2048, 5504)[1] > 1
    assert native.splitk_plan(128, 50264, 2048)[1] == 1
