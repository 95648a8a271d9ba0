"""Sharded FSDP checkpoints: written by 2 gloo ranks, resumed by 3, against one process that never stopped.

The reference has no sharded checkpoints (its FSDP run skips periodic checkpoints and saves no optimizer state,
train.py:251,283); the single-file side of the format is covered by tests/test_core_cpu.py.
"""
import os
import socket
import tempfile

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

CFG = dict(vocab_size=157, context_length=16, d_model=64, num_layers=2, num_heads=4, d_ff=136, rope_theta=10000.0)
SAMPLES = 6          # divisible by both world sizes


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _batch(step):
    g = torch.Generator().manual_seed(11 + step)
    return (torch.randint(0, CFG["vocab_size"], (SAMPLES, 16), generator=g),
            torch.randint(0, CFG["vocab_size"], (SAMPLES, 16), generator=g))


def _steps(wrapped, opt, rank, world, steps):
    per = SAMPLES // world
    for s in steps:
        x, y = _batch(s)
        wrapped.zero_grad()
        wrapped.loss(x[rank * per:(rank + 1) * per], y[rank * per:(rank + 1) * per]).backward()
        if world > 1:
            wrapped.finish_gradient_synchronization()
        opt.step()


def _phase(rank, world, port, directory, steps, resume, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from llm_systems_from_scratch_b200.models.transformer import TransformerLM
        from llm_systems_from_scratch_b200.optim import FusedAdamW
        from llm_systems_from_scratch_b200.parallel import FSDP
        from llm_systems_from_scratch_b200.utils import checkpoint as ckpt
        torch.manual_seed(0 if not resume else 123)      # a resumed run must not depend on its fresh initialisation
        wrapped = FSDP(TransformerLM(**CFG, use_custom_triton=True))
        opt = FusedAdamW(wrapped.parameters(), lr=1e-2, weight_decay=0.1)
        if resume:
            it = ckpt.load_sharded(wrapped, opt, directory)
            assert it == 2
            assert opt._flat[0]["t"] == 3              # two updates done: the next one is the third
        _steps(wrapped, opt, rank, world, steps)
        if not resume:
            ckpt.save_sharded(wrapped, opt, 2, directory)
            assert os.path.exists(os.path.join(directory, f"shard_{rank:05d}.pt"))
        sd = wrapped.full_state_dict()                   # collective
        if rank == 0 and out_path:
            torch.save(sd, out_path)
    finally:
        dist.destroy_process_group()


def test_sharded_checkpoint_resumes_on_another_world_size():
    from llm_systems_from_scratch_b200.models.transformer import TransformerLM
    from llm_systems_from_scratch_b200.optim import FusedAdamW
    torch.manual_seed(0)
    ref_model = TransformerLM(**CFG, use_custom_triton=True)
    ref_opt = FusedAdamW(ref_model.parameters(), lr=1e-2, weight_decay=0.1)
    _steps(ref_model, ref_opt, 0, 1, [0, 1, 2])
    ref = {k: v.clone() for k, v in ref_model.state_dict().items()}
    with tempfile.TemporaryDirectory() as d:
        ck, out = os.path.join(d, "sharded"), os.path.join(d, "final.pt")
        mp.spawn(_phase, args=(2, _free_port(), ck, [0, 1], False, None), nprocs=2, join=True)
        assert sorted(os.listdir(ck)) == ["manifest.json", "shard_00000.pt", "shard_00001.pt"]
        mp.spawn(_phase, args=(3, _free_port(), ck, [2], True, out), nprocs=3, join=True)
        got = torch.load(out)
    assert set(got) == set(ref)
    for k in ref:
        # weights, both moments and the step count all enter the third update: any of them restored wrongly shows here
        assert torch.allclose(got[k], ref[k], atol=3e-4, rtol=1e-4), (k, (got[k] - ref[k]).abs().max().item())
