"""Paged decode attention, KV append and the serving engine on the GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("heads,dh,splits", [(4, 128, 1), (4, 128, 5), (6, 64, 3), (16, 128, 0)])
def test_paged_decode_matches_reference(heads, dh, splits):
    from llm_systems_from_scratch_b200.ops import serving_ops, torch_impl
    d, page, n_pages, r = heads * dh, 16, 64, 5
    g = torch.Generator(device="cuda").manual_seed(0)
    kc = torch.randn(n_pages, page, d, device="cuda", generator=g).bfloat16()
    vc = torch.randn(n_pages, page, d, device="cuda", generator=g).bfloat16()
    qkv = torch.randn(r, 3 * d, device="cuda", generator=g).bfloat16()
    lens = torch.tensor([1, 16, 17, 100, 191], dtype=torch.int32, device="cuda")
    tables = torch.stack([torch.randperm(n_pages, device="cuda", generator=g)[:12] for _ in range(r)]).int()
    out = serving_ops.paged_decode_attention(qkv, kc, vc, tables, lens, heads, splits)
    ref = torch_impl.paged_decode_attention(qkv[:, :d].float(), kc.float(), vc.float(), tables.cpu(), lens.cpu(), heads)
    assert (out.float() - ref).abs().max().item() < 2e-2


def test_kv_append_writes_only_selected_slots():
    from llm_systems_from_scratch_b200.ops import serving_ops
    d = 512
    kc = torch.zeros(8, 16, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    qkv = torch.randn(4, 3 * d, device="cuda").bfloat16()
    slots = torch.tensor([5, -1, 127, 16], device="cuda")
    serving_ops.kv_append(kc, vc, qkv, slots)
    kf, vf = kc.view(-1, d), vc.view(-1, d)
    for i, s in enumerate(slots.tolist()):
        if s >= 0:
            assert torch.equal(kf[s], qkv[i, d:2 * d]) and torch.equal(vf[s], qkv[i, 2 * d:])
    assert int((kf.abs().sum(-1) > 0).sum()) == 3


def test_paged_kernels_report_bad_tables_instead_of_reading_them():
    """A page id beyond the cache, a length beyond the table and a slot beyond the cache are skipped and recorded in
    the status word; good rows of the same launch are unaffected and the context stays usable."""
    from llm_systems_from_scratch_b200.ops import native, serving_ops, torch_impl
    heads, dh, page, n_pages, r = 4, 128, 16, 32, 3
    d = heads * dh
    g = torch.Generator(device="cuda").manual_seed(0)
    kc = torch.randn(n_pages, page, d, device="cuda", generator=g).bfloat16()
    vc = torch.randn(n_pages, page, d, device="cuda", generator=g).bfloat16()
    qkv = torch.randn(r, 3 * d, device="cuda", generator=g).bfloat16()
    tables = torch.stack([torch.randperm(n_pages, device="cuda", generator=g)[:4] for _ in range(r)]).int()
    good_lens = torch.tensor([10, 33, 64], dtype=torch.int32, device="cuda")
    ref = torch_impl.paged_decode_attention(qkv[:, :d].float(), kc.float(), vc.float(), tables.cpu(), good_lens.cpu(), heads)
    native.status_word().zero_()
    for bad_tables, bad_lens in ((tables.clone().index_put_((torch.tensor([1]), torch.tensor([0])), torch.tensor(n_pages + 7, dtype=torch.int32, device="cuda")), good_lens),
                                 (tables, torch.tensor([10, 33, 4 * page + 1], dtype=torch.int32, device="cuda"))):
        out = serving_ops.paged_decode_attention(qkv, kc, vc, bad_tables, bad_lens, heads, 2)
        torch.cuda.synchronize()
        with pytest.raises(native.KernelError):
            native.check_status()
        assert (out[0].float() - ref[0]).abs().max().item() < 2e-2       # the untouched row is still right
        assert torch.isfinite(out.float()).all()
    before = kc.clone()
    serving_ops.kv_append(kc, vc, qkv, torch.tensor([3, n_pages * page, -1], device="cuda"))
    torch.cuda.synchronize()
    with pytest.raises(native.KernelError):
        native.check_status()
    changed = (kc.view(-1, d) != before.view(-1, d)).any(-1).nonzero().flatten().tolist()
    assert changed == [3]
    native.check_status()                                                 # cleared; nothing pending


@pytest.mark.parametrize("graphs", [False, True])
def test_engine_matches_full_recompute_on_gpu(graphs):
    from llm_systems_from_scratch_b200.models.transformer import TransformerLM
    from llm_systems_from_scratch_b200.ops import native
    from llm_systems_from_scratch_b200.serving import ServingEngine
    torch.manual_seed(0)
    cfg = dict(vocab_size=503, context_length=256, d_model=256, num_layers=2, num_heads=4, d_ff=688, rope_theta=10000.0)
    model = TransformerLM(**cfg, use_custom_triton=True).cuda().eval()
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 503, (n,), generator=g).tolist() for n in (5, 130, 33, 64, 17)]
    eng = ServingEngine(model, page_size=16, max_batch=4, max_context=256, use_cuda_graphs=graphs)
    got = eng.generate(prompts, 12)
    native.check_status()
    # oracle: greedy decoding by re-running the same bf16 kernels on the whole context each time
    agree = total = 0
    for p, out in zip(prompts, got):
        ids = torch.tensor([p], device="cuda")
        for tok in out:
            logits = model(ids)[0, -1].float()
            top2 = logits.topk(2).values
            if (top2[0] - top2[1]).item() > 0.05:          # skip numerically tied positions
                total += 1
                agree += int(int(logits.argmax()) == tok)
            ids = torch.cat((ids, torch.tensor([[tok]], device="cuda")), dim=1)
    assert total > 20 and agree == total, (agree, total)
    assert eng.cache.allocator.free == eng.cache.num_pages


@pytest.mark.parametrize("graphs", [False, True])
def test_engine_with_programmatic_dependent_launch_gives_the_same_tokens(graphs):
    """The decode-path kernels launched as programmatic dependents (each starts while the kernel before it drains and
    waits for it before touching global memory) must produce exactly the tokens of ordinary launches, eagerly and in
    captured graphs, and leave the status word clean."""
    from llm_systems_from_scratch_b200.models.transformer import TransformerLM
    from llm_systems_from_scratch_b200.ops import native
    from llm_systems_from_scratch_b200.serving import ServingEngine
    torch.manual_seed(0)
    cfg = dict(vocab_size=503, context_length=256, d_model=256, num_layers=3, num_heads=4, d_ff=688, rope_theta=10000.0)
    model = TransformerLM(**cfg, use_custom_triton=True).cuda().eval()
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 503, (n,), generator=g).tolist() for n in (7, 120, 40, 64, 19, 90)]
    outs = {}
    prev = native.set_pdl(False)
    try:
        for pdl in (False, True):
            native.set_pdl(pdl)
            eng = ServingEngine(model, page_size=16, max_batch=4, max_context=256, use_cuda_graphs=graphs)
            outs[pdl] = eng.generate(prompts, 24)
            torch.cuda.synchronize()
            native.check_status()
            assert eng.cache.allocator.free == eng.cache.num_pages
    finally:
        native.set_pdl(prev)
    assert outs[True] == outs[False]


@pytest.mark.parametrize("heads,dh", [(4, 128), (6, 64), (16, 128)])
def test_rope_kv_append_equals_the_two_separate_kernels(heads, dh):
    from llm_systems_from_scratch_b200.models.transformer import RotaryEmbedding
    from llm_systems_from_scratch_b200.ops import native, serving_ops
    d, page, n_pages, r = heads * dh, 16, 12, 37
    g = torch.Generator(device="cuda").manual_seed(3)
    cache = RotaryEmbedding._build_cache(300, dh, 10000.0).cuda().contiguous()
    qkv = torch.randn(r, 3 * d, device="cuda", generator=g).bfloat16()
    pos = torch.randint(0, 300, (r,), device="cuda", generator=g).int()
    slots = torch.randperm(n_pages * page, device="cuda", generator=g)[:r].long()
    slots[3] = -1
    slots[11] = -1
    a_qkv, b_qkv = qkv.clone(), qkv.clone()
    ka, va = (torch.zeros(n_pages, page, d, device="cuda", dtype=torch.bfloat16) for _ in range(2))
    kb, vb = torch.zeros_like(ka), torch.zeros_like(va)
    native.rope_(a_qkv, cache, pos, heads)
    serving_ops.kv_append(ka, va, a_qkv, slots)
    serving_ops.rope_kv_append(b_qkv, cache, pos, kb, vb, slots, heads)
    torch.cuda.synchronize()
    native.check_status()
    assert torch.equal(a_qkv, b_qkv) and torch.equal(ka, kb) and torch.equal(va, vb)
    # a slot beyond the cache is reported and not written; the row is still rotated
    bad = slots.clone()
    bad[5] = n_pages * page + 9
    c_qkv, kc, vc = qkv.clone(), torch.zeros_like(ka), torch.zeros_like(va)
    serving_ops.rope_kv_append(c_qkv, cache, pos, kc, vc, bad, heads)
    torch.cuda.synchronize()
    with pytest.raises(native.KernelError):
        native.check_status()
    assert torch.equal(c_qkv, a_qkv)
    keep = torch.ones(r, dtype=torch.bool, device="cuda")
    keep[5] = False
    keep &= slots >= 0
    assert torch.equal(kc.view(-1, d)[slots[keep]], ka.view(-1, d)[slots[keep]])
    assert float(kc.view(-1, d)[slots[5]].abs().sum()) == 0.0
