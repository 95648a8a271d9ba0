"""Bandwidth-bound sm_100a kernels against their fp32 PyTorch statements."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, atol, rtol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    lim = atol + rtol * b.abs()
    assert bool((err <= lim).all()), f"max err {err.max().item()} (limit {atol}+{rtol}*|ref|)"


@pytest.mark.parametrize("rows,d", [(64, 512), (1000, 2048), (33, 768), (257, 4096), (16, 1344),
                                    # enough rows for the row-pipelined forward (widths 256 * 1..8) and several
                                    # rows per block in the backward
                                    (4800, 2048), (5003, 768), (6001, 1280), (4737, 256), (5000, 1344)])
def test_rmsnorm_fwd_bwd(rows, d):
    from llm_systems_from_scratch_b200.ops import native, torch_impl
    x = torch.randn(rows, d, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    dy = torch.randn(rows, d, device="cuda").bfloat16()
    y, rstd = native.rmsnorm_fwd(x, w, 1e-5)
    yr, rr = torch_impl.rmsnorm_fwd(x.float(), w.float(), 1e-5)
    _close(y, yr, 2e-2)
    _close(rstd, rr, 1e-4, 1e-4)
    dx, dw = native.rmsnorm_bwd(dy, x, w, rstd)
    dxr, dwr = torch_impl.rmsnorm_bwd(dy.float(), x.float(), w.float(), rr)
    _close(dx, dxr, 3e-2)
    _close(dw, dwr, 1e-2 * math.sqrt(rows), 1e-2)
    dw2 = dw.clone()
    native.rmsnorm_bwd(dy, x, w, rstd, dw_out=dw2, accumulate=True)
    _close(dw2, 2 * dwr, 2e-2 * math.sqrt(rows), 1e-2)
    dres = torch.randn(rows, d, device="cuda").bfloat16()
    dx3, _ = native.rmsnorm_bwd(dy, x, w, rstd, dres=dres)
    _close(dx3, dxr + dres.float(), 4e-2)


@pytest.mark.parametrize("rows,f", [(128, 1344), (1000, 5504), (7, 8)])
def test_silu_mul(rows, f):
    from llm_systems_from_scratch_b200.ops import native, torch_impl
    gu = torch.randn(rows, 2 * f, device="cuda").bfloat16()
    dh = torch.randn(rows, f, device="cuda").bfloat16()
    _close(native.silu_mul_fwd(gu), torch_impl.silu_mul_fwd(gu.float()), 2e-2)
    _close(native.silu_mul_bwd(dh, gu), torch_impl.silu_mul_bwd(dh.float(), gu.float()), 3e-2)


@pytest.mark.parametrize("heads,dh,seq,batch", [(16, 32, 256, 2), (16, 128, 512, 1), (12, 64, 100, 3)])
def test_rope_roundtrip_and_reference(heads, dh, seq, batch):
    from llm_systems_from_scratch_b200.models.transformer import RotaryEmbedding
    from llm_systems_from_scratch_b200.ops import native, torch_impl
    d = heads * dh
    cache = RotaryEmbedding._build_cache(seq + 5, dh, 10000.0).cuda().contiguous()
    qkv = torch.randn(batch * seq, 3 * d, device="cuda").bfloat16()
    pos = (torch.arange(batch * seq, device="cuda") % seq)
    ref = torch_impl.rope_(qkv.float().clone(), cache, pos, heads)
    out = native.rope_(qkv.clone(), cache, None, heads, seq=seq)
    _close(out, ref, 2e-2)
    out2 = native.rope_(qkv.clone(), cache, pos.int().contiguous(), heads)
    assert torch.equal(out, out2)
    back = native.rope_(out.clone(), cache, None, heads, inverse=True, seq=seq)
    _close(back, qkv, 4e-2)
    assert torch.equal(out[:, 2 * d:], qkv[:, 2 * d:])


def test_embedding():
    from llm_systems_from_scratch_b200.ops import native
    v, d, rows = 1000, 512, 4096
    table = torch.randn(v, d, device="cuda").bfloat16()
    tok = torch.randint(0, v, (rows,), device="cuda")
    x = native.embedding_fwd(tok, table)
    assert torch.equal(x, table[tok])
    dx = torch.randn(rows, d, device="cuda").bfloat16()
    g = torch.empty(v, d, device="cuda")
    native.embedding_bwd(dx, tok, g)
    ref = torch.zeros(v, d, device="cuda").index_add_(0, tok, dx.float())
    _close(g, ref, 1e-3, 1e-4)
    # the default path is free of atomics: repeated runs are bitwise identical, also with heavy duplication,
    # accumulation and rows wider than one launch covers
    hot = torch.randint(0, 7, (rows,), device="cuda")
    g1, g2 = torch.empty(v, d, device="cuda"), torch.empty(v, d, device="cuda")
    native.embedding_bwd(dx, hot, g1)
    native.embedding_bwd(dx, hot, g2)
    assert torch.equal(g1, g2)
    _close(g1, torch.zeros(v, d, device="cuda").index_add_(0, hot, dx.float()), 2e-2, 1e-4)
    native.embedding_bwd(dx, tok, g1, accumulate=True)
    _close(g1, g2 + ref, 2e-2, 1e-4)
    ga = torch.empty(v, d, device="cuda")
    native.embedding_bwd(dx, tok, ga, deterministic=False)
    _close(ga, ref, 1e-3, 1e-4)
    wide = torch.randn(64, 5120, device="cuda").bfloat16()
    tw = torch.randint(0, 20, (64,), device="cuda")
    gw = torch.empty(20, 5120, device="cuda")
    native.embedding_bwd(wide, tw, gw)
    _close(gw, torch.zeros(20, 5120, device="cuda").index_add_(0, tw, wide.float()), 1e-2, 1e-4)


@pytest.mark.parametrize("rows,v,ld", [(64, 1000, 1000), (128, 50257, 50264), (16, 10000, 10048)])
def test_xent(rows, v, ld):
    from llm_systems_from_scratch_b200.ops import native, torch_impl
    buf = torch.zeros(rows, ld, device="cuda", dtype=torch.bfloat16)
    buf[:, :v] = (3 * torch.randn(rows, v, device="cuda")).bfloat16()
    logits = buf[:, :v] if ld != v else buf
    tgt = torch.randint(0, v, (rows,), device="cuda")
    tgt[3] = -100
    ref_buf = buf.float().clone()
    ref_loss = torch_impl.xent_fwd_bwd(ref_buf, tgt, 2.0, valid_cols=v)
    loss_only = native.xent_fwd(buf, tgt, valid_cols=v)
    loss = native.xent_fwd_bwd(buf, tgt, 2.0, valid_cols=v)
    assert abs(loss.item() - ref_loss.item()) < 2e-3 * max(1.0, abs(ref_loss.item()))
    assert abs(loss_only.item() - ref_loss.item()) < 2e-3 * max(1.0, abs(ref_loss.item()))
    _close(buf[:, :v], ref_buf[:, :v], 1e-4, 2e-2)
    assert buf[:, v:].abs().max().item() == 0 if ld > v else True
    assert buf[3].abs().max().item() == 0


def test_argmax():
    from llm_systems_from_scratch_b200.ops import native
    x = torch.randn(37, 50264, device="cuda").bfloat16()
    got = native.argmax_rows(x, valid_cols=50257)
    assert torch.equal(got, x[:, :50257].float().argmax(-1))


@pytest.mark.parametrize("n,gdt", [(1 << 20, torch.float32), (12345, torch.bfloat16), (4, torch.float32)])
def test_adamw_matches_reference_order(n, gdt):
    from llm_systems_from_scratch_b200.ops import native, torch_impl
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda").to(gdt)
    m = 0.1 * torch.randn(n, device="cuda")
    v = 0.1 * torch.rand(n, device="cuda")
    mirror = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    scale = torch.tensor(0.5, device="cuda")
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    torch_impl.adamw_step(pr, g, mr, vr, None, 1e-3, 0.9, 0.95, 1e-8, 0.1, 7, grad_scale=scale)
    native.adamw_step(p, g, m, v, mirror, 1e-3, 0.9, 0.95, 1e-8, 0.1, 7, grad_scale=scale)
    _close(p, pr, 1e-6, 1e-5)
    _close(m, mr, 1e-6, 1e-5)
    _close(v, vr, 1e-6, 1e-5)
    assert torch.equal(mirror, p.bfloat16())


def test_sumsq_clip_scale_cast():
    from llm_systems_from_scratch_b200.ops import native
    x = torch.randn(1 << 22, device="cuda")
    s = native.sumsq(x)
    ref = x.double().pow(2).sum().item()
    assert abs(s.item() - ref) / ref < 1e-4
    native.sumsq(x.bfloat16(), out=s)
    assert abs(s.item() - 2 * ref) / ref < 1e-2
    coef = native.clip_coef(torch.tensor(4.0, device="cuda"), 1.0)
    assert abs(coef.item() - 0.5) < 1e-5
    y = x.clone()
    native.scale_(y, coef)
    assert torch.allclose(y, x * coef)
    # unaligned starts and ragged lengths take the scalar head / tail of the vectorised kernel
    for dtype in (torch.float32, torch.bfloat16):
        for off, n in ((1, 1000), (3, 7), (5, 4099), (0, 5)):
            base = torch.randn(8192, device="cuda").to(dtype)
            want = base.clone()
            want[off:off + n] = (base[off:off + n].float() * coef).to(dtype)
            native.scale_(base[off:off + n], coef)
            assert torch.equal(base, want)
    b = torch.empty(x.numel(), device="cuda", dtype=torch.bfloat16)
    native.cast_copy(b, x)
    assert torch.equal(b, x.bfloat16())
    f = torch.empty_like(x)
    native.cast_copy(f, b)
    assert torch.equal(f, b.float())


def test_sample_topk_kernel():
    """Top-k / temperature sampling: support, greedy limit and distribution against the fp32 statement."""
    from llm_systems_from_scratch_b200.ops import native, torch_impl
    torch.manual_seed(0)
    rows, vocab, ld = 64, 50257, 50264
    buf = torch.randn(rows, ld, device="cuda").mul_(3).bfloat16()
    logits = buf[:, :vocab]
    u = torch.rand(rows, device="cuda")
    # top_k = 1 is the argmax whatever the uniform
    top1 = native.sample_topk(logits, u, 0.7, 1)
    assert torch.equal(logits.gather(1, top1[:, None]), logits.gather(1, native.argmax_rows(logits)[:, None]))
    # every draw lies in the top-k set (ties of the k-th value included)
    k = 50
    got = native.sample_topk(logits, u, 1.0, k)
    kth = torch.topk(logits.float(), k, dim=1).values[:, -1]
    assert (logits.float().gather(1, got[:, None])[:, 0] >= kth).all()
    # same inverse-CDF rule as the fp32 statement: identical tokens except where u falls within rounding of a boundary
    ref = torch_impl.sample_topk(logits, u, 1.0, k)
    assert (got == ref).float().mean().item() > 0.9
    # distribution on a small vocabulary: empirical frequencies against softmax probabilities
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0, 3.0, 0.5, -2.0, 1.5]], device="cuda").bfloat16()
    n = 20000
    draws = native.sample_topk(small.expand(n, 8).contiguous(), torch.rand(n, device="cuda"), 0.8, 5)
    freq = torch.bincount(draws, minlength=8).float() / n
    x = small[0].float() / 0.8
    keep = x >= torch.topk(x, 5).values[-1]
    p = torch.softmax(x.masked_fill(~keep, float("-inf")), dim=0)
    assert (freq - p).abs().max().item() < 0.015
    assert freq[~keep].sum().item() == 0
    native.check_status()


@pytest.mark.parametrize("rows,d", [(4800, 2048), (5003, 768), (1184, 256), (6001, 1280), (16384, 2048)])
def test_rmsnorm_bwd_variants_agree(rows, d):
    """Both backward kernels (a block per row with a block-wide reduction; a warp per row) against the fp32 statement,
    with and without the residual gradient; each is bitwise reproducible from run to run."""
    from llm_systems_from_scratch_b200.ops import native, torch_impl
    lib = native.load(required=True)
    g = torch.Generator(device="cuda").manual_seed(rows + d)
    x = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(d, device="cuda", generator=g)).bfloat16()
    dy = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
    dres = torch.randn(rows, d, device="cuda", generator=g).bfloat16()
    _, rstd = native.rmsnorm_fwd(x, w, 1e-5)
    dxr, dwr = torch_impl.rmsnorm_bwd(dy.float(), x.float(), w.float(), rstd)
    got = {}
    old = lib.b200_rmsnorm_set_bwd_rows(0)
    try:
        for v in (0, 1):
            lib.b200_rmsnorm_set_bwd_rows(v)
            dx, dw = native.rmsnorm_bwd(dy, x, w, rstd)
            dx2, dw2 = native.rmsnorm_bwd(dy, x, w, rstd, dres=dres)
            torch.cuda.synchronize()
            native.check_status()
            _close(dx, dxr, 3e-2)
            _close(dx2, dxr + dres.float(), 4e-2)
            _close(dw, dwr, 1e-2 * math.sqrt(rows), 1e-2)
            assert torch.equal(dw, dw2)
            got[v] = (dx, dx2, dw)
    finally:
        lib.b200_rmsnorm_set_bwd_rows(old)
    lib.b200_rmsnorm_set_bwd_rows(1)
    try:
        again = native.rmsnorm_bwd(dy, x, w, rstd)
    finally:
        lib.b200_rmsnorm_set_bwd_rows(old)
    assert torch.equal(again[0], got[1][0]) and torch.equal(again[1], got[1][2])
