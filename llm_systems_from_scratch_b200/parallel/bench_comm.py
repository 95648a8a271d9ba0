"""Roofline measurements of the peer-memory collectives (run under torch.distributed.run).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m llm_systems_from_scratch_b200.parallel.bench_comm [--numel 50593792]

For one FSDP unit of the 1.3B model (50.6 M parameters by default) it times, with CUDA events and the
maximum over ranks, (1) the pull all-gather of bf16 weight shards, (2) the reduce-scatter fused with scale
and sum of squares, (3) the reduce-scatter fused with the AdamW update, (4) the in-place two-shot
all-reduce of an fp32 bucket, and the NCCL collective each one replaces.  The roofline of a kernel is the
slower of its NVLink ingress bytes over the measured 770 GB/s per direction and its HBM bytes over the
measured copy bandwidth; rank 0 prints one JSON line per kernel with achieved / roofline.  It also times
the CTA-pair GEMM that carries the all-gather on its copy warps against the slower of the GEMM at the
measured cuBLAS peak and the gather's NVLink time.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _hbm_gbs() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"])
    except Exception:
        return 6650.0


def _bf16_tflops() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"])
    except Exception:
        return 1590.0


def _time(fn, iters=10, warm=3, reps=4):
    """Median over ``iters`` of the time of ``reps`` back-to-back calls divided by ``reps`` (the ranks' launch
    skew after a host synchronisation is paid once per group, as in a training step), max over ranks."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    best = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        best.append(a.elapsed_time(b) / reps)
    best.sort()
    t = torch.tensor([best[len(best) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--numel", type=int, default=50593792, help="parameters of one unit (1.3B block by default)")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from ..ops import native
    from .peer import PeerComm
    comm = PeerComm()
    ws, rank = comm.world_size, comm.rank
    quantum = ws * 64
    padded = -(-args.numel // quantum) * quantum
    n = padded // ws
    hbm = _hbm_gbs()
    out = []

    def report(name, ms, link_bytes, hbm_bytes, nccl_ms):
        roof_ms = max(link_bytes / NVLINK_GBS, hbm_bytes / hbm) / 1e6
        if rank == 0:
            out.append({"kernel": name, "world": ws, "ms": round(ms, 4), "roofline_ms": round(roof_ms, 4),
                        "fraction_of_roofline": round(roof_ms / ms, 3), "nccl_ms": round(nccl_ms, 4),
                        "nvlink_ingress_mb": round(link_bytes / 1e6, 1)})

    # ---- all-gather of bf16 shards
    shard = comm.alloc(n, torch.bfloat16)
    shard.copy_(torch.randn(n, device="cuda"))
    full = torch.empty(padded, dtype=torch.bfloat16, device="cuda")
    comm.barrier()
    t = _time(lambda: comm.all_gather(full, shard))
    t_n = _time(lambda: dist.all_gather_into_tensor(full, shard))
    report("peer_allgather (bf16 shards)", t, (ws - 1) * n * 2, padded * 2 + n * 2, t_n)

    # ---- the same gather carried by the consumer GEMM (QKV projection shape of the 1.3B block): two copy
    # warps per CTA pull the shards while the MMA warps run.  Roofline: the slower of the GEMM at the measured
    # cuBLAS burst peak and the gather's NVLink bytes; the plain GEMM and gather-then-GEMM are the baselines.
    from .comm import GatherTask
    m_, n_, k_ = 16384, 6144, 2048
    xa = torch.randn(m_, k_, device="cuda").bfloat16()
    wb = torch.randn(n_, k_, device="cuda").bfloat16()
    yc = torch.empty(m_, n_, device="cuda", dtype=torch.bfloat16)
    peak = _bf16_tflops()
    comm.barrier()
    t_plain = _time(lambda: native.gemm(xa, wb, "nt", out=yc, pair=True))

    def fused():
        comm.pre_gather_sync()
        native.gemm(xa, wb, "nt", out=yc, pair=True, gather=GatherTask(comm, full, shard))

    def unfused():
        comm.pre_gather_sync()
        dist.all_gather_into_tensor(full, shard)
        native.gemm(xa, wb, "nt", out=yc, pair=True)
    t_sync = _time(lambda: comm.pre_gather_sync())
    t_f = _time(fused) - t_sync
    t_u = _time(unfused) - t_sync
    flops = 2.0 * m_ * n_ * k_
    roof = max(flops / (peak * 1e12), (ws - 1) * n * 2 / (NVLINK_GBS * 1e9)) * 1e3
    if rank == 0:
        out.append({"kernel": "gemm_bf16_pair carrying the all-gather (16384x6144x2048 + 50.6M bf16 gather)", "world": ws,
                    "ms": round(t_f, 4), "roofline_ms": round(roof, 4), "fraction_of_roofline": round(roof / t_f, 3),
                    "gemm_alone_ms": round(t_plain, 4), "nccl_gather_then_gemm_ms": round(t_u, 4)})

    # ---- reduce-scatter + scale + sumsq, and reduce-scatter + AdamW
    stage = comm.alloc(padded, torch.bfloat16)
    stage.copy_(torch.randn(padded, device="cuda"))
    grad = torch.empty(n, dtype=torch.float32, device="cuda")
    ss = torch.zeros((), device="cuda")
    comm.barrier()
    t = _time(lambda: comm.reduce_scatter_mean(grad, stage, key="bench", sumsq=ss))
    tmp = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    t_n = _time(lambda: dist.reduce_scatter_tensor(tmp, stage, op=dist.ReduceOp.AVG))
    report("peer_reduce_scatter + scale + sumsq (bf16 -> fp32 shard)", t, (ws - 1) * n * 2, n * 2 + n * 4, t_n)
    p, m, v = (torch.randn(n, device="cuda") for _ in range(3))
    v.abs_()
    mirror = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    t = _time(lambda: comm.reduce_scatter_adamw(stage, "bench", p, m, v, mirror, 1e-4, 0.9, 0.95, 1e-8, 0.1, 5))

    def nccl_then_adamw():
        dist.reduce_scatter_tensor(tmp, stage, op=dist.ReduceOp.AVG)
        native.adamw_step(p, tmp, m, v, mirror, 1e-4, 0.9, 0.95, 1e-8, 0.1, 5)
    t_n = _time(nccl_then_adamw)
    report("peer_reduce_scatter + AdamW (one kernel)", t, (ws - 1) * n * 2, n * 2 + n * 26, t_n)

    # ---- two-shot all-reduce of an fp32 bucket (25 MiB)
    nb = 25 * 1024 * 1024 // 4
    bucket = comm.alloc(nb, torch.float32)
    bucket.copy_(torch.randn(nb, device="cuda"))
    comm.barrier()
    t = _time(lambda: comm.all_reduce_mean(bucket))
    ref = bucket.clone()
    t_n = _time(lambda: dist.all_reduce(ref, op=dist.ReduceOp.AVG))
    chunk = nb * 4 / ws
    report("peer_allreduce two-shot (25 MiB fp32 bucket)", t, (ws - 1) * chunk, (ws + 1) * chunk + nb * 4, t_n)
    torch.cuda.synchronize()
    native.check_status()
    if rank == 0:
        for rec in out:
            print(json.dumps(rec))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
