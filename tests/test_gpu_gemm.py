"""tcgen05 GEMM against an fp32 PyTorch matmul of the same bf16 inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, layout):
    af, bf = a.float(), b.float()
    if layout == "nt":
        return af @ bf.t()
    if layout == "nn":
        return af @ bf
    return af.t() @ bf


def _make(layout, m, n, k, dev):
    g = torch.Generator(device=dev).manual_seed(m * 7 + n * 3 + k)
    if layout == "nt":
        a = torch.randn(m, k, device=dev, generator=g)
        b = torch.randn(n, k, device=dev, generator=g)
    elif layout == "nn":
        a = torch.randn(m, k, device=dev, generator=g)
        b = torch.randn(k, n, device=dev, generator=g)
    else:
        a = torch.randn(k, m, device=dev, generator=g)
        b = torch.randn(k, n, device=dev, generator=g)
    return a.bfloat16(), b.bfloat16()


def _check(out, ref, k):
    err = (out.float() - ref).abs().max().item()
    # accumulation error grows with sqrt(k); a bf16 result adds half an ulp of the largest value on top
    tol = 2e-2 * (k ** 0.5) + ref.abs().max().item() * 2.0 ** -8 if out.dtype == torch.bfloat16 else 1e-3 * (k ** 0.5)
    assert err <= tol, f"max abs err {err} > {tol}"


@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (384, 768, 1024), (1000, 1336, 520),
                                   (136, 72, 72), (2048, 5504, 2048)])
def test_gemm_layouts(layout, bn, shape):
    from llm_systems_from_scratch_b200.ops import native
    m, n, k = shape
    a, b = _make(layout, m, n, k, "cuda")
    out = native.gemm(a, b, layout, out_dtype=torch.float32, bn_hint=bn)
    native.check_status()
    _check(out, _ref(a, b, layout), k)
    out16 = native.gemm(a, b, layout, bn_hint=bn)
    native.check_status()
    _check(out16, _ref(a, b, layout), k)


def test_gemm_residual_and_accumulate():
    from llm_systems_from_scratch_b200.ops import native
    m, n, k = 512, 1024, 768
    a, b = _make("nt", m, n, k, "cuda")
    res = torch.randn(m, n, device="cuda").bfloat16()
    out = native.gemm(a, b, "nt", residual=res)
    native.check_status()
    _check(out, _ref(a, b, "nt") + res.float(), k)
    # in-place residual: out aliases the residual
    buf = res.clone()
    native.gemm(a, b, "nt", out=buf, residual=buf)
    native.check_status()
    _check(buf, _ref(a, b, "nt") + res.float(), k)
    acc = torch.ones(m, n, device="cuda", dtype=torch.float32)
    native.gemm(a, b, "nt", out=acc, accumulate=True)
    native.check_status()
    _check(acc, _ref(a, b, "nt") + 1.0, k)


def test_gemm_strided_views_and_auto_tile():
    from llm_systems_from_scratch_b200.ops import native
    m, k = 640, 512
    big = torch.randn(m, 3 * k, device="cuda").bfloat16()
    a = big[:, k:2 * k]                      # row stride 3k, offset k
    w = torch.randn(1344, k, device="cuda").bfloat16()
    out = native.gemm(a, w, "nt")
    native.check_status()
    _check(out, a.float() @ w.float().t(), k)
    outbuf = torch.zeros(m, 2 * 1344, device="cuda", dtype=torch.bfloat16)
    native.gemm(a, w, "nt", out=outbuf[:, 1344:])
    native.check_status()
    _check(outbuf[:, 1344:], a.float() @ w.float().t(), k)
    assert outbuf[:, :1344].abs().max().item() == 0


def test_gemm_many_tiles_persistent():
    from llm_systems_from_scratch_b200.ops import native
    m, n, k = 4096, 4096, 512
    a, b = _make("nt", m, n, k, "cuda")
    out = native.gemm(a, b, "nt")
    native.check_status()
    _check(out, _ref(a, b, "nt"), k)
    # fewer CTAs than tiles forces several tiles per CTA and accumulator double-buffering
    out2 = native.gemm(a, b, "nt", max_ctas=5)
    native.check_status()
    assert torch.equal(out, out2)


@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 768, 512), (1000, 1336, 520), (136, 264, 72), (2048, 5504, 2048),
                                   (4096, 4096, 1024)])
def test_gemm_cta_pair_kernel(layout, shape):
    """cta_group::2 kernel (256 x 256 tiles on CTA pairs) against fp32 matmul and the single-CTA kernel."""
    from llm_systems_from_scratch_b200.ops import native
    m, n, k = shape
    a, b = _make(layout, m, n, k, "cuda")
    out = native.gemm(a, b, layout, out_dtype=torch.float32, pair=True)
    native.check_status()
    _check(out, _ref(a, b, layout), k)
    single = native.gemm(a, b, layout, out_dtype=torch.float32, pair=False)
    assert torch.allclose(out, single, atol=1e-3 * k ** 0.5, rtol=1e-3)
    res = torch.randn(m, n, device="cuda").bfloat16()
    out16 = native.gemm(a, b, layout, residual=res, pair=True)
    native.check_status()
    _check(out16, _ref(a, b, layout) + res.float(), k)


@pytest.mark.parametrize("layout", ["nt", "tn"])
@pytest.mark.parametrize("shape", [(1024, 1001, 256), (1000, 1336, 520), (2048, 5504, 512), (296, 264, 72)])
def test_gemm_pair_tma_store_matches_direct_store(layout, shape):
    """The TMA-store epilogue (tile staged in shared memory) writes exactly what the direct register stores write:
    bf16, bf16 + residual, fp32 and fp32 accumulate, into a padded output view whose columns beyond N stay untouched."""
    from llm_systems_from_scratch_b200.ops import native
    m, n, k = shape
    if layout == "tn" and n % 8:
        pytest.skip("an MN-major B needs a leading dimension that is a multiple of 8")
    a, b = _make(layout, m, n, k, "cuda")
    ld = -(-n // 8) * 8 + 8
    res = torch.randn(m, n, device="cuda").bfloat16()
    outs = {}
    for tma in (True, False):
        prev = native.set_gemm_tma_store(tma)
        try:
            o16 = torch.full((m, ld), 7.0, device="cuda", dtype=torch.bfloat16)
            native.gemm(a, b, layout, out=o16[:, :n], pair=True)
            r16 = torch.full((m, ld), 7.0, device="cuda", dtype=torch.bfloat16)
            native.gemm(a, b, layout, out=r16[:, :n], residual=res, pair=True)
            o32 = torch.full((m, ld), 7.0, device="cuda", dtype=torch.float32)
            native.gemm(a, b, layout, out=o32[:, :n], pair=True)
            acc = torch.full((m, ld), 3.0, device="cuda", dtype=torch.float32)
            native.gemm(a, b, layout, out=acc[:, :n], accumulate=True, pair=True)
            native.gemm(a, b, layout, out=acc[:, :n], accumulate=True, pair=True)
            native.check_status()
        finally:
            native.set_gemm_tma_store(prev)
        outs[tma] = (o16, r16, o32, acc)
    ref = _ref(a, b, layout)
    o16, r16, o32, acc = outs[True]
    _check(o16[:, :n], ref, k)
    _check(r16[:, :n], ref + res.float(), k)
    _check(o32[:, :n], ref, k)
    _check(acc[:, :n], 2 * ref + 3.0, 4 * k)
    for t, d in zip(outs[True], outs[False]):
        assert torch.equal(t[:, :n], d[:, :n])
        assert (t[:, n:] == (3.0 if t is acc else 7.0)).all()      # padding columns are never written


def test_gemm_pair_pad_writable_rows_not_ending_on_16_bytes():
    """A vocabulary-like N (1001): with ``pad_writable`` the TMA-store epilogue runs and may zero columns up to the
    next 16-byte boundary, nothing beyond; without it the padding is untouched."""
    from llm_systems_from_scratch_b200.ops import native
    m, n, k = 1024, 1001, 256
    a, b = _make("nt", m, n, k, "cuda")
    ref = _ref(a, b, "nt")
    for dtype, edge in ((torch.bfloat16, 1008), (torch.float32, 1004)):
        buf = torch.full((m, 1024), 7.0, device="cuda", dtype=dtype)
        native.gemm(a, b, "nt", out=buf[:, :n], pair=True, pad_writable=True)
        native.check_status()
        _check(buf[:, :n], ref, k)
        pad = buf[:, n:edge]
        assert ((pad == 0) | (pad == 7.0)).all()
        assert (buf[:, edge:] == 7.0).all()
        keep = torch.full((m, 1024), 7.0, device="cuda", dtype=dtype)
        native.gemm(a, b, "nt", out=keep[:, :n], pair=True)
        assert torch.equal(keep[:, :n], buf[:, :n]) and (keep[:, n:] == 7.0).all()


@pytest.mark.parametrize("m,f,k", [(1024, 1408, 512), (2048, 5504, 2048), (1100, 256, 264)])
def test_gemm_swiglu_epilogue(m, f, k):
    """gate|up projection with SiLU(gate)*up in the epilogue against GEMM followed by the stand-alone kernel."""
    from llm_systems_from_scratch_b200.ops import native
    x = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(2 * f, k, device="cuda") / k ** 0.5).bfloat16()
    out = native.gemm_swiglu(x, w)
    assert out is not None
    gu, h = out
    native.check_status()
    ref_gu = native.gemm(x, w, "nt")
    ref_h = native.silu_mul_fwd(ref_gu)
    assert torch.allclose(gu.float(), ref_gu.float(), atol=2e-2, rtol=2e-2)
    assert (gu.float() - (x.float() @ w.float().t())).abs().max().item() < 3e-2 * k ** 0.5 / 8
    assert torch.allclose(h.float(), native.silu_mul_fwd(gu).float(), atol=1e-3, rtol=1e-2)
    assert torch.allclose(h.float(), ref_h.float(), atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("m,f,k", [(1024, 1408, 512), (2048, 5504, 2048), (1100, 264, 136)])
def test_gemm_swiglu_backward_epilogue(m, f, k):
    """dh = dy @ W2 with the SiLU*mul backward in the epilogue against the fp32 statement of the same op and
    against GEMM followed by the stand-alone kernel."""
    from llm_systems_from_scratch_b200.ops import native
    dy = torch.randn(m, k, device="cuda").bfloat16()
    w = (torch.randn(k, f, device="cuda") / k ** 0.5).bfloat16()
    gu = torch.randn(m, 2 * f, device="cuda").bfloat16()
    native.FUSE_SWIGLU_BWD = True       # opt-in path (off by default: slower than the two-kernel path end to end)
    try:
        out = native.gemm_swiglu_bwd(dy, w, gu)
    finally:
        native.FUSE_SWIGLU_BWD = False
    assert out is not None
    native.check_status()
    two_step = native.silu_mul_bwd(native.gemm(dy, w, "nn"), gu)
    assert torch.allclose(out.float(), two_step.float(), atol=2e-2, rtol=2e-2)
    dh = dy.float() @ w.float()
    g, u = gu[:, :f].float(), gu[:, f:].float()
    s = torch.sigmoid(g)
    ref = torch.cat([dh * u * (s + g * s * (1 - s)), dh * g * s], dim=1)
    assert (out.float() - ref).abs().max().item() < 4e-2 * max(1.0, ref.abs().max().item()) / 4


def test_gemm_wait_counter_is_bounded_and_reports():
    """A GEMM whose B operand is announced through a device counter (another kernel is still writing it): with the
    counter never bumped and a 1 ms limit the kernel gives up, records the wait in the status word, frees its tensor
    memory and returns; the context stays usable and the same launch with the counter set computes the product."""
    import ctypes
    from llm_systems_from_scratch_b200.ops import native
    lib = native.load()
    P, I, L, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_uint
    lib.b200_gemm_set_wait_limit_ns.argtypes = [ctypes.c_ulonglong]
    lib.b200_gemm_set_wait_limit_ns.restype = ctypes.c_ulonglong
    m, n, k = 512, 512, 256
    a, b = _make("nt", m, n, k, "cuda")
    out = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = native.status_word()
    status.zero_()

    def launch():
        rc = lib.b200_gemm_bf16_pair_gather(a.data_ptr(), b.data_ptr(), out.data_ptr(), None, m, n, k, k, k, n, 0, 0, 0, 0,
                                            None, None, 0, 0, 0, None, None, counter.data_ptr(), 1, status.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()

    old = lib.b200_gemm_set_wait_limit_ns(1_000_000)
    try:
        launch()
        with pytest.raises(native.KernelError):
            native.check_status()
        assert float(out.float().abs().sum()) == 0.0          # it gave up before producing anything
        counter.fill_(1)
        launch()
        native.check_status()
        _check(out, _ref(a, b, "nt"), k)
    finally:
        lib.b200_gemm_set_wait_limit_ns(old)


@pytest.mark.parametrize("shape", [(128, 2048, 2048), (64, 6144, 2048), (128, 11008, 2048), (128, 2048, 5504),
                                   (256, 2048, 2048), (200, 1000, 320), (1, 2048, 2048), (130, 6152, 2112),
                                   (128, 50264, 2048)])
def test_gemm_split_k_small_m(shape, monkeypatch):
    """Decode-sized GEMMs with K split over CTAs: same result as the fp32 matmul for every epilogue, bitwise the
    same from run to run (the partial tiles are added in slice order whichever CTA arrives last), counters left at
    zero, and the plain kernel's answer within rounding."""
    from llm_systems_from_scratch_b200.ops import native
    m, n, k = shape
    a, b = _make("nt", m, n, k, "cuda")
    ref = _ref(a, b, "nt")
    monkeypatch.setattr(native, "USE_SPLITK", False)
    plain = native.gemm(a, b, "nt")
    monkeypatch.setattr(native, "USE_SPLITK", True)
    monkeypatch.setattr(native, "SPLITK_MIN_K", 0)
    bn, splits = native.splitk_plan(m, n, k)
    assert bn in (64, 128, 256) and 1 <= splits <= 8
    if (m, n, k) in ((128, 2048, 2048), (64, 6144, 2048), (128, 2048, 5504)):
        assert splits > 1          # the shapes this exists for really are split
    out = native.gemm(a, b, "nt")
    _check(out, ref, k)
    # two bf16 roundings of sums taken in different orders: up to one ulp of the largest value apart
    assert (out.float() - plain.float()).abs().max().item() <= 2e-2 * (k ** 0.5) + ref.abs().max().item() * 2.0 ** -7
    for _ in range(3):
        assert torch.equal(native.gemm(a, b, "nt"), out)
    res = torch.randn(m, n, device="cuda").bfloat16()
    _check(native.gemm(a, b, "nt", residual=res), ref + res.float(), k)
    out32 = native.gemm(a, b, "nt", out_dtype=torch.float32)
    _check(out32, ref, k)
    acc = out32.clone()
    native.gemm(a, b, "nt", out=acc, accumulate=True)
    _check(acc, 2 * ref, k)
    # a strided output view (a column block of a wider buffer), as the serving engine's fused projections use
    wide = torch.zeros(m, n + 64, device="cuda", dtype=torch.bfloat16)
    view = wide[:, 32:32 + n] if n % 8 == 0 else wide[:, :n]
    native.gemm(a, b, "nt", out=view)
    _check(view, ref, k)
    assert float(wide[:, n + 32:].abs().sum()) == 0.0 or n % 8 != 0
    torch.cuda.synchronize()
    native.check_status()
    _, counters = native._splitk_scratch(a.device)
    assert int(counters.abs().sum().item()) == 0


@pytest.mark.parametrize("shape,max_ctas", [((128, 2048, 2048), 0), ((64, 6144, 2048), 0), ((256, 2048, 5504), 0),
                                            ((1000, 1336, 520), 5), ((130, 520, 136), 1), ((128, 50264, 2048), 0)])
@pytest.mark.parametrize("pdl", [False, True])
def test_gemm_early_weight_tiles_give_the_same_result(shape, max_ctas, pdl):
    """``b_stable`` lets the kernel request its first weight tiles before it waits for the kernel ahead of it; the
    result must be bitwise that of the ordinary order, also when a CTA walks several tiles and when K is split."""
    from llm_systems_from_scratch_b200.ops import native
    m, n, k = shape
    a, b = _make("nt", m, n, k, "cuda")
    res = torch.randn(m, n, device="cuda").bfloat16()
    prev = native.set_pdl(pdl)
    try:
        want = native.gemm(a, b, "nt", residual=res, max_ctas=max_ctas, pair=False)
        for _ in range(3):
            a2 = a.clone()      # a fresh producer kernel right before the GEMM: the wait has something to wait for
            got = native.gemm(a2, b, "nt", residual=res, max_ctas=max_ctas, pair=False, b_stable=True)
            assert torch.equal(got, want)
        torch.cuda.synchronize()
        native.check_status()
    finally:
        native.set_pdl(prev)
    _check(want, _ref(a, b, "nt") + res.float(), k)
