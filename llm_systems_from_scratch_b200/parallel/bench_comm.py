"""Roofline measurements of the peer-memory collectives (run under torch.distributed.run).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m llm_systems_from_scratch_b200.parallel.bench_comm [--numel 50593792]

For one FSDP unit of the 1.3B model (50.6 M parameters by default) it times, with CUDA events and the
maximum over ranks, (1) the pull all-gather of bf16 weight shards, (2) the reduce-scatter fused with scale
and sum of squares, (3) the reduce-scatter fused with the AdamW update, (4) the in-place two-shot
all-reduce of an fp32 bucket, and the NCCL collective each one replaces.  The roofline of a kernel is the
slower of its NVLink ingress bytes over the link bandwidth and its HBM bytes over the measured copy
bandwidth; rank 0 prints one JSON line per kernel with achieved / roofline against two link figures: the
peer-copy bandwidth measured by this same program (first row: every rank pulls 256 MiB from its right-hand
neighbour, once with the copy engine and once with this package's copy kernel) and the nominal 900 GB/s per
direction.  It also times the CTA-pair GEMMs that carry the all-gather or the reduce-scatter (+ AdamW) on
their copy warps against the slower of the GEMM at the measured cuBLAS peak and the collective's NVLink time.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_NOMINAL_GBS = 900.0


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

    class _Out(list):
        def append(self, rec):          # rank 0 prints every record as soon as it exists
            super().append(rec)
            print(json.dumps(rec), flush=True)
    out = _Out()

    # ---- link bandwidth as this box delivers it: every rank pulls 256 MiB from its right-hand neighbour
    probe_n = 256 << 20
    probe_src = comm.alloc(probe_n, torch.uint8)
    probe_dst = torch.empty(probe_n, dtype=torch.uint8, device="cuda")
    peer_ptr = comm._find(probe_src)["peers"][(rank + 1) % ws]
    comm.barrier()
    import ctypes
    cudart = ctypes.CDLL("libcudart.so.12") if ws > 1 else None

    def copy_engine():
        # cudaMemcpyAsync(dst, src, n, cudaMemcpyDefault = 4, stream)
        rc = cudart.cudaMemcpyAsync(ctypes.c_void_p(probe_dst.data_ptr()), ctypes.c_void_p(peer_ptr),
                                    ctypes.c_size_t(probe_n), 4, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0, rc

    def copy_kernel():
        native._check(comm.lib.b200_peer_copy(probe_dst.data_ptr(), peer_ptr, probe_n, 296, comm._stream()), "peer_copy")
    t_ce = _time(copy_engine, reps=2)
    t_ck = _time(copy_kernel, reps=2)
    link_ce, link_sm = probe_n / t_ce / 1e6, probe_n / t_ck / 1e6
    link = max(link_ce, link_sm)          # GB/s per direction per GPU, measured here
    if rank == 0:
        out.append({"kernel": "peer copy probe (256 MiB pulled from the neighbour)", "world": ws,
                    "copy_engine_gbs": round(link_ce, 1), "copy_kernel_gbs": round(link_sm, 1),
                    "nominal_gbs": NVLINK_NOMINAL_GBS})

    def report(name, ms, link_bytes, hbm_bytes, nccl_ms, **extra):
        roof_ms = max(link_bytes / link, hbm_bytes / hbm) / 1e6
        roof_nom = max(link_bytes / NVLINK_NOMINAL_GBS, hbm_bytes / hbm) / 1e6
        if rank == 0:
            out.append({"kernel": name, "world": ws, "ms": round(ms, 4), "roofline_ms": round(roof_ms, 4),
                        "fraction_of_roofline": round(roof_ms / ms, 3),
                        "fraction_of_roofline_nominal_900": round(roof_nom / ms, 3), "nccl_ms": round(nccl_ms, 4),
                        "nvlink_ingress_mb": round(link_bytes / 1e6, 1), **extra})

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
    roof = max(flops / (peak * 1e12), (ws - 1) * n * 2 / (link * 1e9)) * 1e3
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

    # ---- the same two kernels with the staging bound to an NVLink multicast object (NVLS): one multimem.ld_reduce per
    # 16 bytes, the switch adds the copies.  Link bytes per GPU are the same (every GPU still sends 7/8 of its staging
    # into the switch), so the roofline does not move; the SMs issue an eighth of the loads.
    comm.nvls = os.environ.get("B200_NVLS", "1") == "1"
    stage_mc = comm.alloc_multicast(padded, torch.bfloat16)
    if comm.nvls:
        stage_mc.copy_(stage)
        comm.barrier()
        t = _time(lambda: comm.reduce_scatter_mean(grad, stage_mc, key="bench_mc", sumsq=ss))
        report("NVLS reduce-scatter + scale + sumsq (multimem.ld_reduce)", t, (ws - 1) * n * 2, n * 2 + n * 4, float("nan"))
        t = _time(lambda: comm.reduce_scatter_adamw(stage_mc, "bench_mc", p, m, v, mirror, 1e-4, 0.9, 0.95, 1e-8, 0.1, 5))
        report("NVLS reduce-scatter + AdamW (one kernel)", t, (ws - 1) * n * 2, n * 2 + n * 26, float("nan"))

    # ---- the same two reduce-scatters carried by the GEMM that follows a block's backward in FSDP (the dgrad of the
    # gate|up projection, 16384 x 2048 x 11008): one kernel, the copy warps reduce while the MMA warps compute.
    # Roofline: the slower of the GEMM at the measured cuBLAS burst peak and the reduce-scatter's NVLink time.
    m2, n2, k2 = 16384, 2048, 11008
    xa2 = torch.randn(m2, k2, device="cuda").bfloat16()
    wb2 = torch.randn(k2, n2, device="cuda").bfloat16()
    yc2 = torch.empty(m2, n2, device="cuda", dtype=torch.bfloat16)
    comm.barrier()
    t_plain2 = _time(lambda: native.gemm(xa2, wb2, "nn", out=yc2, pair=True))
    flops2 = 2.0 * m2 * n2 * k2
    adam_kw = dict(master=p, m=m, v=v, mirror=mirror, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=5)
    for label, mk, nccl_fn in (
            ("reduce-scatter + scale + sumsq", lambda: comm.reduce_task(stage, "bench", out_shard=grad, sumsq=ss),
             lambda: dist.reduce_scatter_tensor(tmp, stage, op=dist.ReduceOp.AVG)),
            ("reduce-scatter + AdamW", lambda: comm.reduce_task(stage, "bench", sumsq=ss, adamw=adam_kw), nccl_then_adamw)):
        t_c = _time(lambda: native.gemm(xa2, wb2, "nn", out=yc2, pair=True, reduce=mk()))

        def nccl_then_gemm():
            nccl_fn()
            native.gemm(xa2, wb2, "nn", out=yc2, pair=True)
        t_n2 = _time(nccl_then_gemm)
        roof2 = max(flops2 / (peak * 1e12), (ws - 1) * n * 2 / (link * 1e9)) * 1e3
        if rank == 0:
            out.append({"kernel": f"gemm_bf16_pair carrying the {label} (16384x2048x11008 GEMM + 50.6M-parameter unit)",
                        "world": ws, "ms": round(t_c, 4), "roofline_ms": round(roof2, 4),
                        "fraction_of_roofline": round(roof2 / t_c, 3), "gemm_alone_ms": round(t_plain2, 4),
                        "nccl_then_gemm_ms": round(t_n2, 4)})

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
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
