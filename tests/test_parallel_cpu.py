"""DDP and FSDP wrappers on 2-3 CPU ranks (gloo) against single-process training on the full batch."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

CFG = dict(vocab_size=157, context_length=16, d_model=64, num_layers=3, num_heads=4, d_ff=136, rope_theta=10000.0)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _batch(world, per_rank=2, seq=16, seed=5):
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(0, CFG["vocab_size"], (world * per_rank, seq), generator=g)
    y = torch.randint(0, CFG["vocab_size"], (world * per_rank, seq), generator=g)
    return x, y


def _single_process_reference(world, steps, native, clip, delayed=False):
    """Full-batch training in one process.  ``delayed``: scale each step's gradients by the clip coefficient of the
    *previous* step's norm (1 at the first step), which is what the fused reduce-scatter -> AdamW path does."""
    from llm_systems_from_scratch_b200.models.transformer import TransformerLM
    from llm_systems_from_scratch_b200.ops import functional as Fn
    from llm_systems_from_scratch_b200.optim import FusedAdamW
    torch.manual_seed(0)
    model = TransformerLM(**CFG, use_custom_triton=native)
    opt = FusedAdamW(model.parameters(), lr=1e-2, weight_decay=0.1)
    coef = 1.0
    for s in range(steps):
        x, y = _batch(world, seed=5 + s)
        model.zero_grad()
        model.loss(x, y).backward()
        if clip and delayed:
            grads = [p.grad for p in model.parameters() if p.grad is not None]
            norm = torch.sqrt(sum((g.double() ** 2).sum() for g in grads)).item()
            for g in grads:
                g.mul_(coef)
            coef = min(1.0, clip / (norm + 1e-6))
        elif clip:
            Fn.clip_gradient(model.parameters(), clip)
        opt.step()
    return {k: v.clone() for k, v in model.state_dict().items()}


def _worker(rank, world, port, mode, native, steps, clip, out_path, fused=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from llm_systems_from_scratch_b200.models.transformer import TransformerLM
        from llm_systems_from_scratch_b200.ops import functional as Fn
        from llm_systems_from_scratch_b200.optim import FusedAdamW
        from llm_systems_from_scratch_b200.parallel import DDP, FSDP
        torch.manual_seed(rank)            # different init per rank: the wrapper must broadcast rank 0's
        model = TransformerLM(**CFG, use_custom_triton=native)
        if rank == 0:
            torch.manual_seed(0)
            model = TransformerLM(**CFG, use_custom_triton=native)
        # fuse_gather=True exercises the deferred-gather bookkeeping (on CPU the GEMM simply runs the gather first)
        wrapped = DDP(model, bucket_size_mb=0.05) if mode == "ddp" else FSDP(model, fuse_gather=(world == 3))
        opt = FusedAdamW(wrapped.parameters(), lr=1e-2, weight_decay=0.1)
        if fused:
            assert wrapped.attach_optimizer(opt, clip or None)
        per = 2
        for s in range(steps):
            x, y = _batch(world, seed=5 + s)
            xs, ys = x[rank * per:(rank + 1) * per], y[rank * per:(rank + 1) * per]
            wrapped.zero_grad()
            wrapped.loss(xs, ys).backward()
            wrapped.finish_gradient_synchronization()
            if fused:
                norm = wrapped.finish_fused_step()
                assert torch.isfinite(norm)
            elif clip:
                Fn.clip_gradient(wrapped.parameters(), clip)
            opt.step()
        sd = wrapped.full_state_dict() if mode == "fsdp" else model.state_dict()
        if rank == 0:
            torch.save({k: v.clone() for k, v in sd.items()}, out_path)
        if mode == "ddp":
            n_buckets = len(wrapped._buckets)
            assert n_buckets >= 2, n_buckets
    finally:
        dist.destroy_process_group()


def _run(mode, native, world, steps=3, clip=0.0, fused=False):
    port = _free_port()
    with tempfile.TemporaryDirectory() as d:
        out = os.path.join(d, "sd.pt")
        mp.spawn(_worker, args=(world, port, mode, native, steps, clip, out, fused), nprocs=world, join=True)
        got = torch.load(out)
    ref = _single_process_reference(world, steps, native, clip, delayed=fused)
    assert set(got) == set(ref)
    for k in ref:
        assert torch.allclose(got[k], ref[k], atol=3e-4, rtol=1e-4), (k, (got[k] - ref[k]).abs().max().item())
    return got


def test_ddp_arena_mode_matches_single_process():
    _run("ddp", native=True, world=2)


def test_ddp_generic_mode_matches_single_process():
    _run("ddp", native=False, world=2)


def test_fsdp_matches_single_process():
    _run("fsdp", native=True, world=2)


def test_fsdp_three_ranks_with_global_clipping():
    _run("fsdp", native=True, world=3, steps=2, clip=0.25)


def test_fsdp_fused_optimizer_matches_single_process():
    """AdamW inside each unit's reduce-scatter (host statement of the fused kernel on gloo ranks), no clipping:
    the same weights as single-process training."""
    _run("fsdp", native=True, world=2, steps=3, fused=True)


def test_fsdp_fused_optimizer_delayed_clip():
    """With clipping the fused path scales step t by the coefficient of step t-1's norm: it must match a
    single-process run that does exactly that (20 steps, 3 ranks), and stay close to exact clipping."""
    got = _run("fsdp", native=True, world=3, steps=20, clip=0.5, fused=True)
    exact = _single_process_reference(3, 20, True, 0.5, delayed=False)
    worst = max((got[k] - exact[k]).abs().max().item() for k in exact)
    mean = sum((got[k] - exact[k]).abs().sum().item() for k in exact) / sum(v.numel() for v in exact.values())
    # lr 1e-2 for 20 Adam steps can move a weight by 0.2; the one-step lag of the clip factor moves single weights by
    # about half of that at most and the average weight by far less
    assert 0 < worst < 0.2 and mean < 0.03, (worst, mean)


def test_fsdp_world_size_one_aliases_shards():
    from llm_systems_from_scratch_b200.models.transformer import TransformerLM
    from llm_systems_from_scratch_b200.optim import FusedAdamW
    from llm_systems_from_scratch_b200.parallel import FSDP
    torch.manual_seed(0)
    model = TransformerLM(**CFG, use_custom_triton=True)
    ref = _single_process_reference(1, 2, True, 0.0)
    f = FSDP(model)
    assert len(f.fsdp_units) == CFG["num_layers"] + 2      # blocks, embedding table, final norm + lm_head
    assert len(list(f.parameters())) == CFG["num_layers"] + 2
    assert all(p.numel() == 0 for p in model.parameters())       # unsharded weights are really released
    opt = FusedAdamW(f.parameters(), lr=1e-2, weight_decay=0.1)
    for s in range(2):
        x, y = _batch(1, seed=5 + s)
        f.zero_grad()
        f.loss(x, y).backward()
        f.finish_gradient_synchronization()
        opt.step()
    got = f.full_state_dict()
    for k in ref:
        assert torch.allclose(got[k], ref[k], atol=3e-4, rtol=1e-4), k
    logits = f(x)
    assert logits.shape == (2, 16, CFG["vocab_size"])


def test_flag_protocol_model_checker():
    """Random interleavings of the ready / done flag protocol of the peer reduce-scatter: no read of a stale or
    overwritten staging buffer, no deadlock; without the wait on `done` (one unit, so nothing else orders the
    next write after the peers' reads) the checker must find the race."""
    from llm_systems_from_scratch_b200.parallel.protocol_check import ProtocolViolation, check_reduce_scatter_protocol
    for seed in range(200):
        check_reduce_scatter_protocol(world=2 + seed % 4, units=1 + seed % 3, steps=3, seed=seed)
    for seed in range(30):      # the world size of the flagship configuration
        check_reduce_scatter_protocol(world=8, units=1 + seed % 3, steps=3, seed=1000 + seed)
    found = 0
    for seed in range(200):
        try:
            check_reduce_scatter_protocol(world=4, units=1, steps=3, seed=seed, use_wait_readers=False)
        except ProtocolViolation:
            found += 1
    assert found > 0


def test_allreduce_and_weight_gather_protocols():
    """The two other flag protocols under random interleavings: the two-shot in-place all-reduce (a chunk is read only
    while it holds local gradients, consumed only when reduced) and the FSDP weight shards (gathers of step s read
    version s - 1 and never overlap an update; gather slots are not refilled while in use).  Each checker must also
    find the race when the wait that prevents it is taken out."""
    from llm_systems_from_scratch_b200.parallel.protocol_check import (ProtocolViolation, check_allreduce_protocol,
                                                                     check_weight_gather_protocol)
    for seed in range(150):
        check_allreduce_protocol(world=2 + seed % 4, buckets=1 + seed % 3, steps=3, seed=seed)
        check_weight_gather_protocol(world=2 + seed % 4, units=1 + seed % 4, steps=3, seed=seed,
                                     fused_update=bool(seed % 2))
    for seed in range(20):
        check_allreduce_protocol(world=8, buckets=1 + seed % 3, steps=3, seed=2000 + seed)
        check_weight_gather_protocol(world=8, units=1 + seed % 4, steps=3, seed=2000 + seed, fused_update=bool(seed % 2))
    found_ar = found_w = 0
    for seed in range(100):
        try:
            check_allreduce_protocol(world=4, buckets=1, steps=3, seed=seed, wait_for_pushes=False)
        except ProtocolViolation:
            found_ar += 1
        try:
            check_weight_gather_protocol(world=4, units=2, steps=3, seed=seed, await_weights=False)
        except ProtocolViolation:
            found_w += 1
    assert found_ar > 0 and found_w > 0
