"""Micro-benchmarks of the hand-written kernels (CUDA-event timing, L2 flushed between iterations).

    python -m llm_systems_from_scratch_b200.ops.bench_ops gemm            # training GEMM shapes vs cuBLAS
    python -m llm_systems_from_scratch_b200.ops.bench_ops attention       # FlashAttention fwd/bwd vs SDPA
    python -m llm_systems_from_scratch_b200.ops.bench_ops elementwise     # bandwidth-bound kernels vs the copy roofline
    python -m llm_systems_from_scratch_b200.ops.bench_ops gemm-small      # one small GEMM, three launches (for ncu)
    python -m llm_systems_from_scratch_b200.ops.bench_ops gemm-pair-small # three launches of the CTA-pair GEMM (for ncu)
    python -m llm_systems_from_scratch_b200.ops.bench_ops attention-small # one small attention fwd+bwd (for ncu)
    python -m llm_systems_from_scratch_b200.ops.bench_ops attention-trace # in-kernel timeline of one CTA per kernel
    python -m llm_systems_from_scratch_b200.ops.bench_ops decode [ctx]    # serving decode step vs its memory roofline
    python -m llm_systems_from_scratch_b200.ops.bench_ops paged-decode-small  # paged decode attention alone (for ncu)

Each line of output is one JSON record.  The "-small" modes exist so that a profiler capture ends by
itself in seconds: inputs are larger than L2 but only a few hundred MB.
"""
from __future__ import annotations

import json
import sys

import torch

from . import attention, native


def timeit(fn, iters: int = 10, warm: int = 3, flush: bool = True) -> float:
    """Median milliseconds of ``fn`` over ``iters`` runs; L2 is replaced between runs.

    The flush writes a 256 MB buffer and then reads another one: after the write alone L2 is full of *dirty* lines,
    and the timed kernel would pay for their write-back (up to 126 MB of DRAM writes, about 20 us) on top of its own
    traffic - a cost that belongs to the flush, not to the kernel.  After the read pass L2 holds clean, unrelated lines."""
    scrub = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    clean = torch.zeros(64 << 20, dtype=torch.float32, device="cuda") if flush else None
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if scrub is not None:
            scrub.zero_()
            clean.sum()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]


def _operands(layout, m, n, k):
    if layout == "nt":
        return torch.randn(m, k, device="cuda").bfloat16(), torch.randn(n, k, device="cuda").bfloat16()
    if layout == "nn":
        return torch.randn(m, k, device="cuda").bfloat16(), torch.randn(k, n, device="cuda").bfloat16()
    return torch.randn(k, m, device="cuda").bfloat16(), torch.randn(k, n, device="cuda").bfloat16()


GEMM_SHAPES = [("nt", 16384, 6144, 2048), ("nt", 16384, 2048, 2048), ("nt", 16384, 11008, 2048),
               ("nt", 16384, 2048, 5504), ("nn", 16384, 2048, 6144), ("nn", 16384, 2048, 11008),
               ("nn", 16384, 5504, 2048), ("tn", 6144, 2048, 16384), ("tn", 11008, 2048, 16384),
               ("tn", 2048, 5504, 16384), ("nt", 16384, 50264, 2048), ("nt", 8192, 8192, 8192),
               ("nt", 64, 6144, 2048), ("nt", 64, 2048, 5504), ("nt", 64, 50264, 2048)]


def bench_gemm():
    for layout, m, n, k in GEMM_SHAPES:
        a, b = _operands(layout, m, n, k)
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        t = timeit(lambda: native.gemm(a, b, layout, out=out, pair=False))
        t_pair = timeit(lambda: native.gemm(a, b, layout, out=out, pair=True)) if m >= 256 else float("nan")
        t_direct = float("nan")
        if m >= 256:        # the same kernel with direct register stores in the epilogue instead of TMA stores
            prev = native.set_gemm_tma_store(False)
            t_direct = timeit(lambda: native.gemm(a, b, layout, out=out, pair=True))
            native.set_gemm_tma_store(prev)
        ref = {"nt": lambda: torch.matmul(a, b.t(), out=out), "nn": lambda: torch.matmul(a, b, out=out),
               "tn": lambda: torch.matmul(a.t(), b, out=out)}[layout]
        t2 = timeit(ref)
        native.check_status()
        flops = 2.0 * m * n * k
        print(json.dumps({"op": "gemm", "layout": layout, "m": m, "n": n, "k": k, "ms": round(t, 4),
                          "tflops": round(flops / t / 1e9, 1), "pair_ms": round(t_pair, 4),
                          "pair_tflops": round(flops / t_pair / 1e9, 1),
                          "pair_direct_store_tflops": round(flops / t_direct / 1e9, 1), "cublas_ms": round(t2, 4),
                          "cublas_tflops": round(flops / t2 / 1e9, 1)}), flush=True)


def bench_gemm_decode():
    """The GEMMs of one decode step of the 1.3B model (QKV, output, gate|up, down projections of 24 layers; lm_head)
    at batch 64 / 128 / 256: the plain single-CTA kernel, the same kernel with K split over CTAs where the launcher
    would split, and torch.matmul (cuBLAS), against the time the weights alone need at the measured copy bandwidth.

    CUDA events resolve about 2 us here, so a single 10 - 20 us kernel cannot be timed on its own: each figure is a
    CUDA graph of 24 launches of the shape, every launch with its own weight matrix (24 layers; 0.2 - 1.1 GB per
    shape, larger than L2), divided by 24."""
    shapes = [("qkv", 6144, 2048, 24), ("out", 2048, 2048, 24), ("gate_up", 11008, 2048, 24), ("down", 2048, 5504, 24),
              ("lm_head", 50264, 2048, 4)]
    weights = {name: [torch.randn(n, k, device="cuda").bfloat16() for _ in range(reps)] for name, n, k, reps in shapes}

    def graph_us(fn, ws):
        for w in ws[:2]:
            fn(w)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for w in ws:
                fn(w)
        return timeit(g.replay, iters=10, warm=2) * 1e3 / len(ws)

    for m in (64, 128, 256):
        tot = {"plain": 0.0, "splitk": 0.0, "cublas": 0.0}
        for name, n, k, reps in shapes:
            a = torch.randn(m, k, device="cuda").bfloat16()
            out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
            prev = native.USE_SPLITK
            native.USE_SPLITK = False
            t_plain = graph_us(lambda w: native.gemm(a, w, "nt", out=out), weights[name])
            native.USE_SPLITK = True
            native.SPLITK_MIN_K = 0
            t_split = graph_us(lambda w: native.gemm(a, w, "nt", out=out), weights[name])
            native.USE_SPLITK = prev
            native.SPLITK_MIN_K = native.SPLITK_MIN_K_DEFAULT
            t_lib = graph_us(lambda w: torch.matmul(a, w.t(), out=out), weights[name])
            native.check_status()
            bn, splits = native.splitk_plan(m, n, k)
            w_us = n * k * 2 / 6541.8e3
            per_step = 1 if name == "lm_head" else 24
            for key, t in (("plain", t_plain), ("splitk", t_split), ("cublas", t_lib)):
                tot[key] += per_step * t / 1e3
            print(json.dumps({"op": "gemm-decode", "name": name, "m": m, "n": n, "k": k, "split_tile_n": bn,
                              "k_slices": splits, "plain_us": round(t_plain, 2), "splitk_us": round(t_split, 2),
                              "cublas_us": round(t_lib, 2), "weights_at_copy_bw_us": round(w_us, 2)}), flush=True)
        print(json.dumps({"op": "gemm-decode-step", "m": m, "layers": 24,
                          **{k + "_ms": round(v, 3) for k, v in tot.items()}}), flush=True)


def bench_attention():
    for b, s, h, dh in [(8, 2048, 16, 128), (16, 1024, 12, 64), (2, 4096, 32, 128)]:
        qkv = torch.randn(b * s, 3 * h * dh, device="cuda").bfloat16()
        flops = 4.0 * b * h * s * s * dh / 2
        o, lse = attention.attention_fwd(qkv, b, s, h)
        do = torch.randn_like(o)
        t_f = timeit(lambda: attention.attention_fwd(qkv, b, s, h))
        t_b = timeit(lambda: attention.attention_bwd(do, qkv, o, lse, b, s, h))
        q, k, v = (x.reshape(b, s, h, dh).transpose(1, 2).detach().requires_grad_() for x in
                   qkv.view(b * s, 3, h * dh).unbind(1))
        oo = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
        g = torch.randn_like(oo)
        t_sf = timeit(lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True))
        t_sb = timeit(lambda: torch.autograd.grad(oo, (q, k, v), g, retain_graph=True))
        native.check_status()
        print(json.dumps({"op": "attention", "shape": [b, s, h, dh], "fwd_ms": round(t_f, 4),
                          "fwd_tflops": round(flops / t_f / 1e9, 1), "bwd_ms": round(t_b, 4),
                          "bwd_tflops": round(2.5 * flops / t_b / 1e9, 1), "sdpa_fwd_ms": round(t_sf, 4),
                          "sdpa_bwd_ms": round(t_sb, 4)}), flush=True)


def bench_elementwise():
    rows, d, f = 16384, 2048, 5504
    x = torch.randn(rows, d, device="cuda").bfloat16()
    w = torch.ones(d, device="cuda").bfloat16()
    dy = torch.randn_like(x)
    dres = torch.randn_like(x)
    gu = torch.randn(rows, 2 * f, device="cuda").bfloat16()
    dh = torch.randn(rows, f, device="cuda").bfloat16()
    _, rstd = native.rmsnorm_fwd(x, w, 1e-5)
    n = 64 << 20
    p, g, m, v = (torch.randn(n, device="cuda") for _ in range(4))
    v.abs_()
    mirror = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    lib = native.load(required=True)

    def fwd_per_block():       # the general-width kernel (one block per eight rows), for comparison
        lib.b200_rmsnorm_set_fwd_rows(0)
        native.rmsnorm_fwd(x, w, 1e-5)
        lib.b200_rmsnorm_set_fwd_rows(1)

    def bwd_variant(v):        # 0: a block per row, block-wide reduction; 1: a warp per row
        def run():
            old = lib.b200_rmsnorm_set_bwd_rows(v)
            native.rmsnorm_bwd(dy, x, w, rstd, dres=dres)
            lib.b200_rmsnorm_set_bwd_rows(old)
        return run

    cases = [("rmsnorm_fwd", lambda: native.rmsnorm_fwd(x, w, 1e-5), 2 * x.numel() * 2),
             ("rmsnorm_fwd_general_width_kernel", fwd_per_block, 2 * x.numel() * 2),
             ("rmsnorm_bwd", lambda: native.rmsnorm_bwd(dy, x, w, rstd, dres=dres), 4 * x.numel() * 2),
             ("rmsnorm_bwd_general_width_kernel", bwd_variant(0), 4 * x.numel() * 2),
             ("rmsnorm_bwd_no_residual", lambda: native.rmsnorm_bwd(dy, x, w, rstd), 3 * x.numel() * 2),
             ("silu_mul_fwd", lambda: native.silu_mul_fwd(gu), 3 * rows * f * 2),
             ("silu_mul_bwd", lambda: native.silu_mul_bwd(dh, gu), 5 * rows * f * 2),
             ("adamw", lambda: native.adamw_step(p, g, m, v, mirror, 1e-3, 0.9, 0.95, 1e-8, 0.1, 3), n * 30)]
    for name, fn, nbytes in cases:
        t = timeit(fn)
        print(json.dumps({"op": name, "ms": round(t, 4), "gb_per_s": round(nbytes / t / 1e6, 1)}), flush=True)


def gemm_small():
    a, b = _operands("nt", 8192, 6144, 2048)
    out = torch.empty(8192, 6144, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        native.gemm(a, b, "nt", out=out, bn_hint=256)
    torch.cuda.synchronize()
    native.check_status()
    print(json.dumps({"op": "gemm-small", "ok": True}))


def gemm_pair_small():
    a, b = _operands("nt", 8192, 6144, 2048)
    out = torch.empty(8192, 6144, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        native.gemm(a, b, "nt", out=out, pair=True)
    torch.cuda.synchronize()
    native.check_status()
    print(json.dumps({"op": "gemm-pair-small", "ok": True}))


def attention_small():
    b, s, h, dh = 4, 2048, 16, 128
    qkv = torch.randn(b * s, 3 * h * dh, device="cuda").bfloat16()
    o, lse = attention.attention_fwd(qkv, b, s, h)
    do = torch.randn_like(o)
    for _ in range(2):
        attention.attention_fwd(qkv, b, s, h)
        attention.attention_bwd(do, qkv, o, lse, b, s, h)
    torch.cuda.synchronize()
    native.check_status()
    print(json.dumps({"op": "attention-small", "ok": True}))


def attention_trace():
    """Per-step timeline (SM clock stamps) of one CTA of each attention kernel: where each role waits."""
    import ctypes
    lib = native.load()
    b, s, h, dh = 8, 2048, 16, 128
    qkv = torch.randn(b * s, 3 * h * dh, device="cuda").bfloat16()
    o, lse = attention.attention_fwd(qkv, b, s, h)
    do = torch.randn_like(o)
    attention.attention_bwd(do, qkv, o, lse, b, s, h)
    torch.cuda.synchronize()

    def capture(setter, cta, fn):
        buf = torch.zeros(10 * 64 * 8, dtype=torch.int64, device="cuda")
        setter(ctypes.c_void_p(buf.data_ptr()), cta)
        fn()
        torch.cuda.synchronize()
        setter(ctypes.c_void_p(0), 0)
        t = buf.cpu().view(10, 64, 8)
        base = int(t[t > 0].min())
        return [[[int(v) - base if v > 0 else None for v in t[role, step]] for step in range(20)] for role in range(10)]

    fwd = lambda: attention.attention_fwd(qkv, b, s, h)
    bwd = lambda: attention.attention_bwd(do, qkv, o, lse, b, s, h)
    # CTA 200 is a mid-grid CTA with many steps in all three kernels; a negative index selects the dK/dV kernel
    for name, setter, cta, fn, roles in (("flash_fwd", lib.b200_flash_fwd_set_trace, 200, fwd, (1, 2, 6)),
                                         ("flash_dq", lib.b200_flash_bwd_set_trace, 200, bwd, (0, 1, 2, 6)),
                                         ("flash_dkdv", lib.b200_flash_bwd_set_trace, -201, bwd, (1, 2, 6))):
        rec = capture(setter, cta, fn)
        for role in roles:
            for step in (6, 7, 8):
                print(json.dumps({"op": "attention-trace", "kernel": name, "role": role, "step": step,
                                  "clk": rec[role][step]}), flush=True)
    native.check_status()


def bench_decode(argv=()):
    """Decode step of the 1.3B serving model against its memory roofline, per batch bucket.

    A decode step must read every weight once (2.84 GB in bf16) and every cached K / V byte of the running requests
    once; roofline = those bytes over the measured copy bandwidth.  Reports the whole engine step (host preparation,
    H2D of the step's inputs, graph replay, D2H of the sampled tokens), the device time of the graph alone, and the
    paged-attention kernel and the small-M GEMMs on their own."""
    import os
    from ..models.transformer import TransformerLM
    from ..serving import Request, ServingEngine
    from . import serving_ops
    ctx = int(argv[0]) if argv else 1200
    hbm = 6541.8
    try:
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            hbm = float(json.load(f)["hbm_gbs"])
    except Exception:
        pass
    cfg = dict(vocab_size=50257, context_length=2048, d_model=2048, num_layers=24, num_heads=16, d_ff=5504, rope_theta=10000.0)
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = TransformerLM(**cfg, use_flash_attn=True, use_custom_triton=True)
    model.eval()
    weight_bytes = 2 * (cfg["num_layers"] * (4 * 2048 * 2048 + 3 * 2048 * 5504) + 50257 * 2048)
    g = torch.Generator().manual_seed(1)
    for batch in (32, 64, 128, 256):
        eng = ServingEngine(model, num_pages=batch * (-(-(ctx + 400) // 16)) + 8, page_size=16, max_batch=batch,
                            max_context=2048)
        reqs = [Request(i, torch.randint(0, 50257, (ctx,), generator=g).tolist(), 400) for i in range(batch)]
        for r in reqs:
            eng.sched.add(r)
        eng._realtime, eng._virtual = False, float("inf")
        while eng.sched.waiting:
            eng.step(float("inf"))
        running = list(eng.sched.running)
        assert len(running) == batch, (len(running), batch)
        for _ in range(3):
            eng.decode(running)
        torch.cuda.synchronize()
        import time
        t0 = time.perf_counter()
        n_it = 20
        for _ in range(n_it):
            eng.decode(running)
        torch.cuda.synchronize()
        step_ms = (time.perf_counter() - t0) / n_it * 1e3
        st = eng._graphs[eng._bucket(batch)]
        dev_ms = timeit(lambda: st["graph"].replay(), iters=10, warm=2, flush=False)
        # the engine's own loop: the step is launched before the previous step's tokens have reached the host
        for _ in range(3):
            eng.step(float("inf"))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n_it):
            eng.step(float("inf"))
        torch.cuda.synchronize()
        pipe_ms = (time.perf_counter() - t0) / n_it * 1e3
        kv_bytes = sum(r.context_len for r in running) * 2 * 2048 * 2 * cfg["num_layers"]
        roof_ms = (weight_bytes + kv_bytes) / hbm / 1e6
        # the attention kernel of one layer on the same tables
        qkv = torch.randn(eng._bucket(batch), 3 * 2048, device="cuda").bfloat16()
        att_ms = timeit(lambda: serving_ops.paged_decode_attention(qkv, eng.cache.k[0], eng.cache.v[0], st["tables"],
                                                                   st["ctx"], 16, st["splits"]), iters=10, warm=2)
        print(json.dumps({"op": "decode-step", "batch": batch, "context": ctx, "engine_step_ms": round(pipe_ms, 3),
                          "blocking_step_ms": round(step_ms, 3), "graph_ms": round(dev_ms, 3),
                          "roofline_ms": round(roof_ms, 3), "fraction_of_roofline": round(roof_ms / pipe_ms, 3),
                          "tok_per_s": round(batch / pipe_ms * 1e3),
                          "paged_attention_layer_ms": round(att_ms, 4),
                          "paged_attention_gbs": round(kv_bytes / cfg["num_layers"] / att_ms / 1e6, 1)}), flush=True)
        del eng, st
        torch.cuda.empty_cache()
    for m in (32, 64, 128, 256):
        for n, k in ((6144, 2048), (2048, 2048), (11008, 2048), (2048, 5504), (50264, 2048)):
            a = torch.randn(m, k, device="cuda").bfloat16()
            b = torch.randn(n, k, device="cuda").bfloat16()
            out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
            t = timeit(lambda: native.gemm(a, b, "nt", out=out))
            t2 = timeit(lambda: torch.matmul(a, b.t(), out=out))
            print(json.dumps({"op": "gemm-decode", "m": m, "n": n, "k": k, "us": round(t * 1e3, 1),
                              "weight_gbs": round(n * k * 2 / t / 1e6, 1),
                              "cublas_us": round(t2 * 1e3, 1)}), flush=True)
    native.check_status()


def paged_decode_small():
    """Three launches of the paged decode attention on a cache larger than L2 (batch 64, 1024 cached tokens per
    request, 16 heads of 128: 268 MB of K and 268 MB of V are read per launch); small enough for a profiler."""
    from . import serving_ops
    heads, dh, page, batch, ctx = 16, 128, 16, 64, 1024
    d = heads * dh
    n_pages = batch * ctx // page
    kc = torch.randn(n_pages, page, d, device="cuda").bfloat16()
    vc = torch.randn(n_pages, page, d, device="cuda").bfloat16()
    qkv = torch.randn(batch, 3 * d, device="cuda").bfloat16()
    tables = torch.randperm(n_pages, device="cuda").int().view(batch, ctx // page).contiguous()
    lens = torch.full((batch,), ctx, dtype=torch.int32, device="cuda")
    splits = serving_ops.choose_splits(batch, heads, ctx)
    for _ in range(3):
        serving_ops.paged_decode_attention(qkv, kc, vc, tables, lens, heads, splits)
    torch.cuda.synchronize()
    native.check_status()
    t = timeit(lambda: serving_ops.paged_decode_attention(qkv, kc, vc, tables, lens, heads, splits))
    print(json.dumps({"op": "paged-decode-small", "ms": round(t, 4), "gb_per_s": round(2 * kc.numel() * 2 / t / 1e6, 1),
                      "splits": splits, "ok": True}))


def paged_splits_sweep(argv=()):
    """Paged decode attention of one layer of the 1.3B model (16 heads of 128) at context 1200 for every number of
    context splits from 1 to 32, per batch size: achieved GB/s of K and V, and the number `choose_splits` picks."""
    from . import serving_ops
    heads, dh, page = 16, 128, 16
    d = heads * dh
    ctx = int(argv[0]) if argv else 1200
    for batch in (32, 64, 128, 256):
        pages_per = -(-(ctx + 16) // page)
        n_pages = batch * pages_per + 8
        kc = torch.randn(n_pages, page, d, device="cuda").bfloat16()
        vc = torch.randn(n_pages, page, d, device="cuda").bfloat16()
        qkv = torch.randn(batch, 3 * d, device="cuda").bfloat16()
        tables = torch.zeros(batch, 128, dtype=torch.int32, device="cuda")
        tables[:, :pages_per] = torch.randperm(n_pages, device="cuda")[:batch * pages_per].int().view(batch, pages_per)
        lens = torch.full((batch,), ctx, dtype=torch.int32, device="cuda")
        res = {}
        for s in range(1, 33):
            t = timeit(lambda: serving_ops.paged_decode_attention(qkv, kc, vc, tables, lens, heads, s), iters=10, warm=2)
            res[s] = round(batch * ctx * 2 * d * 2 / t / 1e6)
        native.check_status()
        print(json.dumps({"op": "paged-splits", "batch": batch, "context": ctx,
                          "chosen": serving_ops.choose_splits(batch, heads, 2048, head_dim=dh), "gbs_by_splits": res}),
              flush=True)


def decode_launches(argv=()):
    """One decode step of the 1.3B serving model at a given batch and context with every kernel launched on its own
    (no CUDA graph), bracketed by cudaProfilerStart / Stop: under ``ncu --profile-from-start off`` the capture is
    exactly the launches of that step."""
    from ..models.transformer import TransformerLM
    from ..serving import Request, ServingEngine
    batch = int(argv[0]) if argv else 128
    ctx = int(argv[1]) if len(argv) > 1 else 1200
    cfg = dict(vocab_size=50257, context_length=2048, d_model=2048, num_layers=24, num_heads=16, d_ff=5504, rope_theta=10000.0)
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = TransformerLM(**cfg, use_flash_attn=True, use_custom_triton=True)
    model.eval()
    g = torch.Generator().manual_seed(1)
    eng = ServingEngine(model, num_pages=batch * (-(-(ctx + 64) // 16)) + 8, page_size=16, max_batch=batch,
                        max_context=2048, use_cuda_graphs=False)
    for i in range(batch):
        eng.sched.add(Request(i, torch.randint(0, 50257, (ctx,), generator=g).tolist(), 64))
    eng._realtime, eng._virtual = False, float("inf")
    while eng.sched.waiting:
        eng.step(float("inf"))
    running = list(eng.sched.running)
    for _ in range(2):
        eng.decode(running)
    torch.cuda.synchronize()
    native.reset_launch_count()
    torch.cuda.profiler.start()
    eng.decode(running)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    native.check_status()
    print(json.dumps({"op": "decode-launches", "batch": batch, "context": ctx, "own_launches": native.launch_count(),
                      "split_k": native.USE_SPLITK}))


def main(argv=None):
    argv = argv if argv is not None else sys.argv[1:]
    mode = argv[0] if argv else "gemm"
    if mode == "decode":
        return bench_decode(argv[1:])
    if mode == "decode-launches":
        return decode_launches(argv[1:])
    if mode == "paged-splits":
        return paged_splits_sweep(argv[1:])
    if mode == "paged-decode-small":
        return paged_decode_small()
    {"gemm": bench_gemm, "gemm-decode": bench_gemm_decode, "attention": bench_attention, "elementwise": bench_elementwise, "gemm-small": gemm_small, "gemm-pair-small": gemm_pair_small, "attention-trace": attention_trace,
     "attention-small": attention_small}[mode]()


if __name__ == "__main__":
    main()
