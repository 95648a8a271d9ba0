"""Peer-memory collectives and the FSDP / DDP wrappers on 2+ GPUs (child processes, NCCL for plumbing)."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _spawn(fn, world, *args):
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.spawn(fn, args=(world, _free_port()) + args, nprocs=world, join=True)


def _init(rank, world, port):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")      # no rank leaves in these tests; NCCL is plumbing only
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))


def test_bounded_flag_wait_reports_instead_of_hanging():
    """One GPU: wait on a flag nobody sets, with a 1 ms limit; the kernel returns an error status."""
    import ctypes
    from llm_systems_from_scratch_b200.ops import native
    lib = native.load()
    P, I, U, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_ulonglong
    lib.b200_peer_wait.argtypes = [P, I, U, L, P, P]
    lib.b200_peer_wait.restype = I
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    status = native.status_word()
    status.zero_()
    rc = lib.b200_peer_wait(flags.data_ptr(), 4, 1, 1_000_000, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    with pytest.raises(native.KernelError):
        native.check_status()
    assert int(status[0]) == 0                       # cleared by check_status
    assert float(torch.ones(4, device="cuda").sum()) == 4.0   # the context is still usable


def _collectives(rank, world, port):
    import torch.distributed as dist
    _init(rank, world, port)
    try:
        from llm_systems_from_scratch_b200.ops import native, torch_impl
        from llm_systems_from_scratch_b200.parallel.peer import PeerComm
        comm = PeerComm()
        n = 64 * 1024 + 64
        g = torch.Generator(device="cuda").manual_seed(100 + rank)
        # all-gather of bf16 shards
        shard = comm.alloc(n, torch.bfloat16)
        shard.copy_(torch.randn(n, device="cuda", generator=g))
        comm.barrier()
        full = torch.empty(world * n, dtype=torch.bfloat16, device="cuda")
        comm.all_gather(full, shard)
        ref = torch.empty_like(full)
        dist.all_gather_into_tensor(ref, shard)
        assert torch.equal(full, ref)
        # reduce-scatter (mean) of bf16 staging into fp32 with sum of squares
        stage = comm.alloc(world * n, torch.bfloat16)
        for it in range(3):                          # repeated use exercises the epoch / reuse protocol
            comm.wait_readers(stage, "t")
            stage.copy_(torch.randn(world * n, device="cuda", generator=g))
            out = torch.empty(n, dtype=torch.float32, device="cuda")
            ss = torch.zeros((), device="cuda")
            comm.reduce_scatter_mean(out, stage, key="t", sumsq=ss)
            tmp = stage.float()
            dist.all_reduce(tmp)
            want = tmp[rank * n:(rank + 1) * n] / world
            assert torch.allclose(out, want, atol=1e-6), (out - want).abs().max()
            assert abs(ss.item() - want.pow(2).sum().item()) < 1e-2 * want.pow(2).sum().item()
        # fused reduce-scatter + AdamW against reduce-scatter followed by the AdamW kernel
        comm.wait_readers(stage, "t")
        stage.copy_(torch.randn(world * n, device="cuda", generator=g))
        p0 = torch.randn(n, device="cuda", generator=g)
        m0 = 0.1 * torch.randn(n, device="cuda", generator=g)
        v0 = 0.1 * torch.rand(n, device="cuda", generator=g)
        coef = torch.tensor(0.5, device="cuda")
        tmp = stage.float()
        dist.all_reduce(tmp)
        gref = tmp[rank * n:(rank + 1) * n] / world
        pr, mr, vr = p0.clone(), m0.clone(), v0.clone()
        torch_impl.adamw_step(pr, gref, mr, vr, None, 1e-3, 0.9, 0.95, 1e-8, 0.1, 3, grad_scale=coef)
        p, m, v = p0.clone(), m0.clone(), v0.clone()
        mirror = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        comm.reduce_scatter_adamw(stage, "t", p, m, v, mirror, 1e-3, 0.9, 0.95, 1e-8, 0.1, 3, grad_scale=coef)
        assert torch.allclose(p, pr, atol=1e-6, rtol=1e-5) and torch.allclose(m, mr, atol=1e-6) and torch.allclose(v, vr, atol=1e-6)
        assert torch.equal(mirror, p.bfloat16())
        # the same two reduce-scatters carried on the copy warps of a CTA-pair GEMM (one kernel does both jobs)
        from llm_systems_from_scratch_b200.parallel.comm import GatherTask
        a = torch.randn(2048, 512, device="cuda", generator=g).bfloat16()
        w = torch.randn(1024, 512, device="cuda", generator=g).bfloat16()
        want_c = native.gemm(a, w, "nt", pair=True)
        for it in range(2):
            comm.wait_readers(stage, "t")
            stage.copy_(torch.randn(world * n, device="cuda", generator=g))
            tmp = stage.float()
            dist.all_reduce(tmp)
            want = tmp[rank * n:(rank + 1) * n] / world
            out = torch.zeros(n, dtype=torch.float32, device="cuda")
            ss = torch.zeros((), device="cuda")
            task = comm.reduce_task(stage, "t", out_shard=out, sumsq=ss)
            full2 = torch.zeros_like(full)
            c = native.gemm(a, w, "nt", pair=True, reduce=task, gather=GatherTask(comm, full2, shard))
            assert task.done and torch.equal(c, want_c)
            assert torch.equal(full2, ref)
            assert torch.allclose(out, want, atol=1e-6), (out - want).abs().max()
            assert abs(ss.item() - want.pow(2).sum().item()) < 1e-2 * want.pow(2).sum().item()
        comm.wait_readers(stage, "t")
        stage.copy_(torch.randn(world * n, device="cuda", generator=g))
        tmp = stage.float()
        dist.all_reduce(tmp)
        gref = tmp[rank * n:(rank + 1) * n] / world
        pr, mr, vr = p0.clone(), m0.clone(), v0.clone()
        torch_impl.adamw_step(pr, gref, mr, vr, None, 1e-3, 0.9, 0.95, 1e-8, 0.1, 3, grad_scale=coef)
        p, m, v = p0.clone(), m0.clone(), v0.clone()
        ss = torch.zeros((), device="cuda")
        task = comm.reduce_task(stage, "t", sumsq=ss, adamw=dict(master=p, m=m, v=v, mirror=mirror, lr=1e-3, beta1=0.9,
                                                                 beta2=0.95, eps=1e-8, weight_decay=0.1, step=3,
                                                                 grad_scale=coef))
        c = native.gemm(a, w, "nt", pair=True, reduce=task)
        assert task.done and torch.equal(c, want_c)
        assert torch.allclose(p, pr, atol=1e-6, rtol=1e-5) and torch.allclose(m, mr, atol=1e-6) and torch.allclose(v, vr, atol=1e-6)
        assert torch.equal(mirror, p.bfloat16())
        assert abs(ss.item() - gref.pow(2).sum().item()) < 1e-2 * gref.pow(2).sum().item()
        assert comm.launches.get("reduce_scatter_carried", 0) == 3
        # in-place mean all-reduce of fp32
        buf = comm.alloc(n, torch.float32)
        for it in range(3):
            buf.copy_(torch.randn(n, device="cuda", generator=g))
            want = buf.clone()
            dist.all_reduce(want)
            want /= world
            comm.all_reduce_mean(buf)
            assert torch.allclose(buf, want, atol=1e-6)
        # init-time broadcast: every rank pulls rank 0's tensor (odd byte counts and unaligned views included)
        for numel, dtype, off in ((1 << 20, torch.float32, 0), (12345, torch.bfloat16, 1), (7, torch.float32, 0)):
            base = torch.randn(numel + off, device="cuda", generator=g).to(dtype)
            t = base[off:]
            want = t.clone()
            dist.broadcast(want, src=0)
            comm.PEER_BROADCAST = True
            comm.broadcast(t, src=0)
            assert torch.equal(t, want)
        torch.cuda.synchronize()
        native.check_status()
        comm.check_guards()        # nothing wrote outside a peer-addressable buffer
        # the check itself: a byte written just past a buffer is reported
        probe = comm.alloc(256, torch.uint8)
        band = comm._find(probe)["guards"]
        band[comm.GUARD_BYTES + 256] = 0
        with pytest.raises(RuntimeError, match="guard bytes"):
            comm.check_guards()
        band[comm.GUARD_BYTES + 256] = comm.GUARD_PATTERN
        comm.check_guards()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_collectives_match_nccl(world):
    _spawn(_collectives, world)


def _collectives_nvls(rank, world, port):
    """Reduce-scatter through an NVLink multicast object: the switch adds the ranks' copies (multimem.ld_reduce)."""
    import torch.distributed as dist
    _init(rank, world, port)
    try:
        from llm_systems_from_scratch_b200.ops import native, torch_impl
        from llm_systems_from_scratch_b200.parallel.peer import PeerComm
        comm = PeerComm(nvls=True)
        n = 64 * 1024 + 64
        g = torch.Generator(device="cuda").manual_seed(200 + rank)
        stage = comm.alloc_multicast(world * n, torch.bfloat16)
        if not comm.nvls:
            if rank == 0:
                print("NVLS multicast is not available on this fabric: nothing to test")
            return
        a = torch.randn(2048, 512, device="cuda", generator=g).bfloat16()
        w = torch.randn(1024, 512, device="cuda", generator=g).bfloat16()
        want_c = native.gemm(a, w, "nt", pair=True)
        for it in range(4):
            comm.wait_readers(stage, "t")
            stage.copy_(torch.randn(world * n, device="cuda", generator=g))
            tmp = stage.float()
            dist.all_reduce(tmp)
            want = tmp[rank * n:(rank + 1) * n] / world
            out = torch.zeros(n, dtype=torch.float32, device="cuda")
            ss = torch.zeros((), device="cuda")
            if it % 2 == 0:                         # a kernel of its own
                comm.reduce_scatter_mean(out, stage, key="t", sumsq=ss)
            else:                                   # carried by a GEMM
                task = comm.reduce_task(stage, "t", out_shard=out, sumsq=ss)
                c = native.gemm(a, w, "nt", pair=True, reduce=task)
                assert task.done and torch.equal(c, want_c)
            # the switch returns the sum as bf16 (fp32 accumulation inside): up to one ulp of bf16 on the sum
            assert torch.allclose(out, want, rtol=2.0 ** -7, atol=1e-6), (out - want).abs().max()
            assert abs(ss.item() - want.pow(2).sum().item()) < 2e-2 * want.pow(2).sum().item()
        comm.wait_readers(stage, "t")
        stage.copy_(torch.randn(world * n, device="cuda", generator=g))
        tmp = stage.float()
        dist.all_reduce(tmp)
        gref = tmp[rank * n:(rank + 1) * n] / world
        p0 = torch.randn(n, device="cuda", generator=g)
        m0 = 0.1 * torch.randn(n, device="cuda", generator=g)
        v0 = 0.1 * torch.rand(n, device="cuda", generator=g)
        pr, mr, vr = p0.clone(), m0.clone(), v0.clone()
        torch_impl.adamw_step(pr, gref, mr, vr, None, 1e-3, 0.9, 0.95, 1e-8, 0.1, 3)
        p, m, v = p0.clone(), m0.clone(), v0.clone()
        mirror = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        comm.reduce_scatter_adamw(stage, "t", p, m, v, mirror, 1e-3, 0.9, 0.95, 1e-8, 0.1, 3)
        # the gradient carries up to one bf16 ulp of error: (1 - beta1) of it reaches m, twice its relative size v
        assert torch.allclose(m, mr, rtol=0, atol=0.1 * 2.0 ** -7 * gref.abs().max().item() + 1e-6)
        assert torch.allclose(v, vr, rtol=2.0 ** -5, atol=1e-6)
        assert (p - pr).abs().max().item() < 2e-4
        assert torch.equal(mirror, p.bfloat16())
        assert comm.launches.get("reduce_scatter_nvls", 0) == 5
        torch.cuda.synchronize()
        native.check_status()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_nvls_reduce_scatter_matches_nccl(world):
    _spawn(_collectives_nvls, world)


CFG = dict(vocab_size=1003, context_length=128, d_model=256, num_layers=3, num_heads=4, d_ff=768, rope_theta=10000.0)


def _train(rank, world, port, mode, comm_kind, fused, out):
    import torch.distributed as dist
    _init(rank, world, port)
    try:
        from llm_systems_from_scratch_b200.models.transformer import TransformerLM
        from llm_systems_from_scratch_b200.ops import native
        from llm_systems_from_scratch_b200.optim import FusedAdamW
        from llm_systems_from_scratch_b200.parallel import DDP, FSDP
        torch.manual_seed(0)
        native.FORCE_PAIR = comm_kind == "peer"      # tiny GEMMs on the CTA-pair kernel, which carries the collectives
        model = TransformerLM(**CFG, use_custom_triton=True).cuda()
        wrapped = FSDP(model, comm=comm_kind) if mode == "fsdp" else DDP(model, bucket_size_mb=1.0, comm=comm_kind)
        opt = FusedAdamW(wrapped.parameters(), lr=1e-3, weight_decay=0.1)
        if fused:
            assert wrapped.attach_optimizer(opt, max_grad_norm=0.5)
        arena = wrapped.shard_arena if mode == "fsdp" else model.engine().provider.arena
        losses = []
        for step in range(4):
            g = torch.Generator().manual_seed(7)      # the same batch every step: the loss must go down
            x = torch.randint(0, CFG["vocab_size"], (2 * world, 128), generator=g)[rank * 2:(rank + 1) * 2].cuda()
            y = torch.randint(0, CFG["vocab_size"], (2 * world, 128), generator=g)[rank * 2:(rank + 1) * 2].cuda()
            loss = wrapped.loss(x, y)
            loss.backward()
            wrapped.finish_gradient_synchronization()
            if fused:
                wrapped.finish_fused_step()
            else:
                opt.set_grad_scale(arena.clip_coef(0.5))
            opt.step()
            t = loss.detach().clone()
            dist.all_reduce(t)
            losses.append(t.item() / world)
        torch.cuda.synchronize()
        native.check_status()
        if hasattr(wrapped.comm, "check_guards"):
            wrapped.comm.check_guards()
        state = wrapped.full_state_dict() if mode == "fsdp" else None      # collective
        carried = getattr(wrapped.comm, "launches", {})
        if rank == 0:
            torch.save({"losses": losses, "state": state, "launches": dict(carried)}, out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("mode,fused", [("fsdp", False), ("fsdp", True), ("ddp", False)])
def test_peer_training_matches_nccl_training(tmp_path, mode, fused, world):
    """Four optimizer steps with the peer-memory kernels (collectives carried by GEMMs under FSDP) against the same
    steps with torch.distributed collectives: same losses, same final weights up to the bf16 staging of gradients."""
    a, b = str(tmp_path / "nccl.pt"), str(tmp_path / "peer.pt")
    _spawn(_train, world, mode, "torch", fused, a)
    _spawn(_train, world, mode, "peer", fused, b)
    ra, rb = torch.load(a), torch.load(b)
    la, lb = ra["losses"], rb["losses"]
    assert la[-1] < la[0]
    assert max(abs(p - q) for p, q in zip(la, lb)) < 2e-2, (la, lb)
    if mode == "fsdp":
        # lr 1e-3 for 4 steps moves a weight by at most 4e-3 (Adam steps are sign-like at first, so an element whose
        # tiny gradient rounds differently in the two summation orders may move the other way); on average the runs agree
        for k, v in ra["state"].items():
            diff = (v - rb["state"][k]).abs()
            assert diff.max().item() < 8.1e-3 and diff.mean().item() < 2e-4, (k, diff.max().item(), diff.mean().item())
        assert rb["launches"].get("reduce_scatter_carried", 0) >= 4 * CFG["num_layers"]   # 3 of 5 units per step
        assert rb["launches"].get("all_gather_carried", 0) > 0
