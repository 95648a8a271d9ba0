#!/usr/bin/env python
"""Flagship benchmark: FSDP training throughput of the 1.3B TransformerLM (tokens/s).

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Config (weak scaling): vocab 50,257, d_model 2048, 24 layers, 16 heads, d_ff 5504, context 2048,
micro-batch 8 sequences per GPU, bf16 compute with fp32 sharded AdamW state, global-norm clipping,
synthetic uniform-random token ids, random-init weights.

Two numbers are measured, both on the device with CUDA events and reduced as the max over ranks:

* ``value``     - K full training steps (forward, backward, reduce-scatter, clip, AdamW) on batches
                  that already sit in device memory;
* ``e2e.value`` - the same K steps through the public API a user calls, where every step also copies
                  its batch from pinned host memory to the device and reads the loss back to the host.

``--impl reference`` runs the unmodified reference implementation (installed under baseline/_ref)
through its own public classes on the same config and prints the same JSON line.

Serving (the second half of the headline metric: continuous-batching decode tokens/s and time to first
token of the 1.3B model under a Poisson trace, one replica per GPU):

    python bench.py --workload serve [--gpus N] [--serving-requests 1024]

prints a line of its own (``serving_decode_tok_per_s``).  The default training run appends a short
version of the same measurement (``--serving-requests`` requests, 0 switches it off) under the key
``serving`` of its JSON line, so that one command reports both halves.  The reference has no serving
engine; its arm replays the head of the same trace through its ``TransformerLM`` with a per-request greedy
loop that re-runs the whole context for every token (what its ``generate`` does) for a bounded time.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))

CONFIGS = {
    "fsdp_1p3b": dict(model="TransformerLM-1.3B", vocab_size=50257, context_length=2048, d_model=2048,
                      num_layers=24, num_heads=16, d_ff=5504, rope_theta=10000.0, micro_batch=8),
    "ddp_124m": dict(model="TransformerLM-124M-class", vocab_size=50257, context_length=1024, d_model=768,
                     num_layers=12, num_heads=12, d_ff=2048, rope_theta=10000.0, micro_batch=16),
    "fsdp_7b": dict(model="TransformerLM-7B", vocab_size=32000, context_length=4096, d_model=4096, num_layers=32,
                    num_heads=32, d_ff=11008, rope_theta=10000.0, micro_batch=2, activation_checkpointing=True),
    "tiny": dict(model="TransformerLM-tiny", vocab_size=10000, context_length=256, d_model=512, num_layers=4,
                 num_heads=8, d_ff=1344, rope_theta=10000.0, micro_batch=8),
}

LR, WEIGHT_DECAY, MAX_GRAD_NORM = 3e-4, 0.1, 1.0

# continuous-batching serving of the 1.3B model: Poisson arrivals per GPU, 16-token KV pages, greedy decoding
SERVE = dict(model="TransformerLM-1.3B", vocab_size=50257, context_length=2560, d_model=2048, num_layers=24,
             num_heads=16, d_ff=5504, rope_theta=10000.0, page_size=16, max_batch=256, rate=20.0,
             prompt_len=(128, 2048), output_len=(64, 512))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["native", "reference"], default="native")
    ap.add_argument("--config", choices=sorted(CONFIGS), default="fsdp_1p3b")
    ap.add_argument("--parallel", choices=["fsdp", "ddp"], default="fsdp")
    ap.add_argument("--comm", choices=["auto", "torch", "peer"], default="auto")
    ap.add_argument("--fused-optimizer", choices=["auto", "on", "off"], default="auto",
                    help="FSDP on 2+ GPUs: run AdamW inside each unit's reduce-scatter (clip coefficient from the previous "
                         "step's norm); auto = on from 4 GPUs.  off = reduce-scatter, exact global-norm clip, then one "
                         "AdamW launch")
    ap.add_argument("--nvls", action="store_true",
                    help="gradient staging bound to an NVLink multicast object: the reduce-scatters use multimem.ld_reduce "
                         "(the switch adds the copies) instead of peer loads")
    ap.add_argument("--activation-checkpointing", choices=["config", "on", "off"], default="config",
                    help="per-block activation checkpointing: as the config names it (on for fsdp_7b), or forced")
    ap.add_argument("--workload", choices=["train", "serve"], default="train")
    ap.add_argument("--serving-requests", type=int, default=None,
                    help="requests of the Poisson trace per GPU (serve: default 1024; train: a short serving run of "
                         "this many requests is appended to the line, default 160, 0 = none)")
    ap.add_argument("--serving-time-limit", type=float, default=20.0,
                    help="seconds after which the reference's per-request loop stops")
    ap.add_argument("--seed", type=int, default=0)
    return ap.parse_args()


def init_dist(args):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torch.distributed.run with --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    if world > 1 or args.impl == "reference":
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29512")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))
    return rank, local_rank, world


def l2_policy(cfg) -> str:
    """Every step streams the bf16 weights, the fp32 optimizer state and the saved activations: far more than L2."""
    d, ff, layers, v = cfg["d_model"], cfg["d_ff"], cfg["num_layers"], cfg["vocab_size"]
    params = layers * (4 * d * d + 3 * d * ff + 2 * d) + 2 * v * d + d
    toks = cfg["micro_batch"] * cfg["context_length"]
    acts = toks * layers * (6 * d + 3 * ff) * 2
    return (f"inputs larger than L2 (126 MB): {params * 2 / 1e9:.2f} GB of bf16 weights, {params * 16 / 1e9:.1f} GB of fp32 "
            f"master / moments / gradients and about {acts / 1e9:.1f} GB of saved activations are streamed every step")


def synthetic_tokens(vocab: int, n: int, seed: int):
    import numpy as np
    return np.random.default_rng(seed).integers(0, vocab, size=n, dtype=np.uint32)


def timed_region(step_fn, steps, warmup, world, sampler_gpu):
    """Warm up, then time exactly ``steps`` calls of ``step_fn`` with CUDA events (max over ranks)."""
    import torch
    import torch.distributed as dist
    for _ in range(warmup):
        step_fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    clocks = ClockSampler(sampler_gpu) if sampler_gpu is not None else None
    if clocks:
        clocks.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    t0.record()
    for _ in range(steps):
        step_fn()
    t1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall0
    ms = t0.elapsed_time(t1)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms, wall, (clocks.stop() if clocks else None)


class PeerPathGaveUp(RuntimeError):
    """Raised on every rank together: the peer-memory collectives reported an error during the first step."""


def run_native(args, cfg, rank, local_rank, world):
    import torch
    sys.path.insert(0, ROOT)
    from llm_systems_from_scratch_b200.data import BatchSampler
    from llm_systems_from_scratch_b200.models.transformer import TransformerLM
    from llm_systems_from_scratch_b200.ops import native
    from llm_systems_from_scratch_b200.optim import FusedAdamW
    from llm_systems_from_scratch_b200.parallel import DDP, FSDP

    dev = torch.device("cuda", local_rank)
    if args.nvls:
        os.environ["B200_NVLS"] = "1"
    torch.manual_seed(args.seed)
    mkeys = ("vocab_size", "context_length", "d_model", "num_layers", "num_heads", "d_ff", "rope_theta")
    with torch.device(dev):
        model = TransformerLM(**{k: cfg[k] for k in mkeys}, use_flash_attn=True, use_custom_triton=True)
    ac = bool(cfg.get("activation_checkpointing", False)) if args.activation_checkpointing == "config" else \
        args.activation_checkpointing == "on"
    model.activation_checkpointing = ac
    wrapped = FSDP(model, comm=args.comm) if args.parallel == "fsdp" else DDP(model, comm=args.comm)
    opt = FusedAdamW(wrapped.parameters(), lr=LR, weight_decay=WEIGHT_DECAY)
    # auto: from four ranks on.  On two ranks a rank's shard is half the model and the AdamW pass that the copy warps
    # of a GEMM then carry (658 MB of optimizer state per unit) outlasts the GEMM; there the one-launch AdamW is faster.
    want_fused = args.fused_optimizer == "on" or (args.fused_optimizer == "auto" and world >= 4)
    fused = args.parallel == "fsdp" and world > 1 and want_fused and wrapped.attach_optimizer(opt, MAX_GRAD_NORM)
    arena = wrapped.shard_arena if args.parallel == "fsdp" else model.engine().provider.arena
    b, s = cfg["micro_batch"], cfg["context_length"]
    tokens = synthetic_tokens(cfg["vocab_size"], 1 << 24, args.seed + 1)
    sampler = BatchSampler(tokens, b, s, dev, seed=args.seed, rank=rank)
    loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()
    last = {"loss": None}

    def train_step(x, y):
        wrapped.zero_grad()
        loss = wrapped.loss(x, y)
        loss.backward()
        wrapped.finish_gradient_synchronization()
        if fused:
            wrapped.finish_fused_step()      # the updates ran inside the reduce-scatters; this step's norm clips the next
        else:
            opt.set_grad_scale(arena.clip_coef(MAX_GRAD_NORM))   # global-norm clip folded into the update
        opt.step()
        return loss

    # ---- region A: batches resident on the device (larger than L2 together with the activations)
    pool = [sampler.next() for _ in range(4)]
    it = {"i": 0}

    def step_resident():
        x, y = pool[it["i"] % len(pool)]
        it["i"] += 1
        last["loss"] = train_step(x, y)

    if world > 1 and args.comm == "auto":
        # One untimed step, then all ranks agree on whether any of them saw a device wait run out (a peer that never
        # signalled) or an exception: either every rank goes on, or every rank raises and main() repeats the run
        # on the library collectives and says so in its line.  This covers failures that every rank lives through
        # (a status word set by a bounded wait, an error all ranks raise); a rank that leaves the step early also
        # leaves the step's host collectives unmatched, and that ends in the process group's timeout as before.
        import torch.distributed as dist
        bad = torch.zeros(1, dtype=torch.int32, device=dev)
        why = ""
        try:
            step_resident()
            torch.cuda.synchronize()
            native.check_status()
        except Exception as e:      # noqa: BLE001 - whatever it was, the ranks must leave this step together
            bad.fill_(1)
            why = f"{type(e).__name__}: {str(e)[:120]}"
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad.item()):
            raise PeerPathGaveUp(why or "another rank reported an error")
    native.reset_launch_count()
    comm_counts = getattr(wrapped.comm, "launches", None)
    if comm_counts is not None:
        comm_counts.clear()
    ms, wall, clocks = timed_region(step_resident, args.steps, args.warmup, world, local_rank if rank == 0 else None)
    launches = native.launch_count()
    per_step = lambda n: n * args.steps // max(1, args.steps + args.warmup)
    launches_timed = per_step(launches)
    comm_launches = {k: per_step(v) for k, v in sorted((comm_counts or {}).items())}
    native.check_status()
    loss_a = float(last["loss"].item())

    # ---- region B: end to end (pinned host batch -> device every step, loss read back every step)
    ev = {"e": None}

    def step_e2e():
        x, y = sampler.next()                      # H2D of this step's batch from pinned memory
        loss = train_step(x, y)
        if ev["e"] is not None:
            ev["e"].synchronize()                  # previous step's loss is on the host
            last["host_loss"] = float(loss_host[0])
        loss_host.copy_(loss.detach().reshape(1), non_blocking=True)   # D2H of this step's loss
        e = torch.cuda.Event()
        e.record()
        ev["e"] = e

    ms_e2e, wall_e2e, _ = timed_region(step_e2e, args.steps, 1, world, None)
    native.check_status()
    tokens_per_step = b * s * world
    return dict(ms=ms, ms_e2e=ms_e2e, wall=wall, clocks=clocks, tokens_per_step=tokens_per_step,
                launches=launches_timed, loss=loss_a, h2d=sampler.bytes_per_batch(), d2h=4,
                mem_gb=torch.cuda.max_memory_allocated() / 2 ** 30,
                parallelism=f"{args.parallel}{world}",
                comm=type(wrapped.comm).__name__ + (" + NVLS reduce-scatter" if getattr(wrapped.comm, "nvls", False) else ""),
                comm_launches=comm_launches,
                activation_checkpointing=ac,
                optimizer=("AdamW fp32 sharded state, update fused into each unit's reduce-scatter, global-norm clip 1.0 "
                           "with the previous step's norm" if fused else
                           "AdamW fp32 state, one launch, exact global-norm clip 1.0"))


def run_serving(args, rank, local_rank, world, n_requests):
    """One serving replica on this rank's GPU: the Poisson trace in real time (decode tokens/s, TTFT), then the
    first requests again with arrival times ignored (throughput).  Prompts start as host token lists and every
    sampled token is read back to the host, so the numbers are end to end by construction."""
    import torch
    sys.path.insert(0, ROOT)
    from llm_systems_from_scratch_b200.serving import ServingEngine, poisson_trace
    dev = torch.device("cuda", local_rank)
    keys = ("vocab_size", "context_length", "d_model", "num_layers", "num_heads", "d_ff", "rope_theta")
    trace = poisson_trace(n_requests, SERVE["rate"], SERVE["prompt_len"], SERVE["output_len"], SERVE["vocab_size"],
                          seed=args.seed + rank)
    if args.impl == "reference":
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_dir, "llm_core")):
            return {"unavailable": "reference is not installed under baseline/_ref"}
        sys.path.insert(0, ref_dir)
        from llm_core.model import TransformerLM as RefLM
        from serve import naive_loop
        torch.manual_seed(args.seed)
        model = RefLM(**{k: SERVE[k] for k in keys}, use_flash_attn=True).to(dev).eval()
        res = naive_loop(model, trace, str(dev), args.serving_time_limit)
        del model
        torch.cuda.empty_cache()
        return {"decode_tok_per_s": res["decode_tok_per_s"], "ttft_p50_ms": res["ttft_p50_s"] * 1e3, "ttft_p99_ms": None,
                "requests": res["requests"], "output_tokens": res["output_tokens"], "wall_s": res["wall_s"],
                "offline_tok_per_s": None, "engine": "none: per-request greedy loop over the reference TransformerLM, whole "
                "context re-run per token, stopped after --serving-time-limit seconds", "launches": None}
    from llm_systems_from_scratch_b200.models.transformer import TransformerLM
    from llm_systems_from_scratch_b200.ops import native
    torch.manual_seed(args.seed)
    with torch.device(dev):
        model = TransformerLM(**{k: SERVE[k] for k in keys}, use_flash_attn=True, use_custom_triton=True)
    model.eval()
    eng = ServingEngine(model, page_size=SERVE["page_size"], max_batch=SERVE["max_batch"],
                        max_context=SERVE["context_length"])
    eng.warmup()                                   # decode graphs of every batch bucket are captured before the trace
    eng.generate([trace[0].prompt[:256]], 4)       # one short request end to end: first-launch set-up of the prefill path
    native.reset_launch_count()
    res = eng.run(trace, realtime=True)
    native.check_status()
    launches = native.launch_count()
    off_trace = poisson_trace(min(n_requests, 512), SERVE["rate"], SERVE["prompt_len"], SERVE["output_len"],
                              SERVE["vocab_size"], seed=args.seed + 1000 + rank)
    off = eng.run(off_trace, realtime=False)
    native.check_status()
    out = {"decode_tok_per_s": res["decode_tok_per_s"], "ttft_p50_ms": res["ttft_p50_s"] * 1e3,
           "ttft_p99_ms": res["ttft_p99_s"] * 1e3, "requests": res["requests"], "output_tokens": res["output_tokens"],
           "wall_s": res["wall_s"], "offline_tok_per_s": off["decode_tok_per_s"], "offline_requests": off["requests"],
           "decode_steps": res["decode_steps"], "prefill_tokens": res["prefill_tokens"], "kv_pages": res["kv_pages"],
           "engine": f"continuous batching, paged KV ({SERVE['page_size']}-token pages), max batch {SERVE['max_batch']}, "
                     "CUDA-graphed decode steps", "launches": launches}
    del eng, model
    torch.cuda.empty_cache()
    return out


def gather_serving(rec, world):
    """Whole-job serving record: tokens/s add up over the replicas, TTFT is the median / worst of the replicas'."""
    if world == 1 or rec is None:
        return rec
    import torch.distributed as dist
    allr = [None] * world
    dist.all_gather_object(allr, rec)
    if any("unavailable" in r for r in allr):
        return next(r for r in allr if "unavailable" in r)
    wall = max(r["wall_s"] for r in allr)
    out = dict(allr[0])
    out.update(decode_tok_per_s=sum(r["output_tokens"] for r in allr) / wall, wall_s=wall,
               requests=sum(r["requests"] for r in allr), output_tokens=sum(r["output_tokens"] for r in allr),
               ttft_p50_ms=statistics.median(r["ttft_p50_ms"] for r in allr),
               ttft_p99_ms=None if allr[0]["ttft_p99_ms"] is None else max(r["ttft_p99_ms"] for r in allr),
               offline_tok_per_s=None if allr[0]["offline_tok_per_s"] is None else sum(r["offline_tok_per_s"] for r in allr),
               per_replica_tok_per_s=[round(r["decode_tok_per_s"], 1) for r in allr])
    return out


def serving_config():
    return {"model": SERVE["model"], "arrival": f"Poisson {SERVE['rate']} requests/s per GPU", "prompt_len": list(SERVE["prompt_len"]),
            "output_len": list(SERVE["output_len"]), "page_size": SERVE["page_size"], "decoding": "greedy",
            "replicas": "one data-parallel replica per GPU", "vocab": SERVE["vocab_size"], "d_model": SERVE["d_model"],
            "layers": SERVE["num_layers"], "heads": SERVE["num_heads"], "d_ff": SERVE["d_ff"]}


def run_reference(args, cfg, rank, local_rank, world):
    """The reference's own classes on its stock fastest path: bf16 autocast, SDPA, Triton kernels, its FSDP."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "llm_core")):
        return None, "reference is not installed under baseline/_ref (pip install --target baseline/_ref failed or was not run)"
    sys.path.insert(0, ref_dir)
    import numpy as np
    import torch
    try:
        from llm_core.dataloader import sample_batch
        from llm_core.model import TransformerLM
        from llm_core.nn_functional import clip_gradient
        from llm_systems.kernels.triton_adamw import FusedAdamW
        from llm_systems.kernels.triton_cross_entropy import triton_cross_entropy
        from llm_systems.parallelism.ddp import DDP
        from llm_systems.parallelism.fsdp_zero3 import FSDP
    except Exception as e:  # pragma: no cover
        return None, f"reference import failed: {type(e).__name__}: {e}"
    if "baseline/_ref" not in sys.modules["llm_core"].__file__.replace(os.sep, "/"):
        return None, "llm_core did not resolve to baseline/_ref"

    torch.set_float32_matmul_precision("high")
    dev = f"cuda:{local_rank}"
    torch.manual_seed(args.seed)
    mkeys = ("vocab_size", "context_length", "d_model", "num_layers", "num_heads", "d_ff", "rope_theta")
    model = TransformerLM(**{k: cfg[k] for k in mkeys}, use_flash_attn=True, use_custom_triton=True).to(dev)
    model = FSDP(model) if args.parallel == "fsdp" else DDP(model)
    model.train()
    opt = FusedAdamW(params=model.parameters(), lr=LR, weight_decay=WEIGHT_DECAY)
    b, s = cfg["micro_batch"], cfg["context_length"]
    tokens = synthetic_tokens(cfg["vocab_size"], 1 << 24, args.seed + 1)
    tmp = tempfile.NamedTemporaryFile(suffix=".bin", delete=False)
    tokens.tofile(tmp.name)
    data = np.memmap(tmp.name, dtype=np.uint32, mode="r")
    torch.manual_seed(args.seed + 100 + rank)
    last = {}

    def train_step(x, y):
        model.zero_grad()
        with torch.autocast(device_type="cuda", dtype=torch.bfloat16, enabled=True):
            logits = model(x)
            loss = triton_cross_entropy(logits.view(-1, logits.size(-1)), y.view(-1))
        loss.backward()
        model.finish_gradient_synchronization()
        clip_gradient(model.parameters(), MAX_GRAD_NORM)
        opt.step()
        return loss

    pool = [sample_batch(data, b, s, dev) for _ in range(4)]
    it = {"i": 0}

    def step_resident():
        x, y = pool[it["i"] % len(pool)]
        it["i"] += 1
        last["loss"] = train_step(x, y)

    ms, wall, clocks = timed_region(step_resident, args.steps, args.warmup, world, local_rank if rank == 0 else None)
    loss_a = float(last["loss"].item())

    def step_e2e():
        x, y = sample_batch(data, b, s, dev)        # the reference's loader: pinned host batch -> device
        loss = train_step(x, y)
        last["host_loss"] = loss.item()             # the reference's loop reads the loss every step

    ms_e2e, wall_e2e, _ = timed_region(step_e2e, args.steps, 1, world, None)
    os.unlink(tmp.name)
    return dict(ms=ms, ms_e2e=ms_e2e, wall=wall, clocks=clocks, tokens_per_step=b * s * world, launches=None,
                loss=loss_a, h2d=2 * b * s * 8, d2h=4, mem_gb=torch.cuda.max_memory_allocated() / 2 ** 30,
                parallelism=f"{args.parallel}{world}", comm="NCCL", comm_launches=None, activation_checkpointing=False,
                optimizer="reference FusedAdamW (Triton), clip 1.0 by each rank's local shard norm (the reference's "
                          "clip_gradient over its FSDP shards)" if args.parallel == "fsdp" and world > 1 else
                          "reference FusedAdamW (Triton), global-norm clip 1.0"), None


def main():
    args = parse_args()
    cfg = CONFIGS[args.config]
    try:
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
    except Exception as e:
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": f"no GPU in this process: {e}"}))
            return 0
        raise
    rank, local_rank, world = init_dist(args)
    if args.workload == "serve":
        n_req = args.serving_requests if args.serving_requests is not None else 1024
        clocks = ClockSampler(local_rank) if rank == 0 else None
        if clocks:
            clocks.start()
        rec = gather_serving(run_serving(args, rank, local_rank, world, n_req), world)
        clk = clocks.stop() if clocks else None
        if rank == 0:
            if "unavailable" in rec:
                print(json.dumps({"impl": args.impl, "workload": "serve", "unavailable": rec["unavailable"]}))
            else:
                r1 = lambda v: None if v is None else round(v, 1)
                print(json.dumps({
                    "metric": "serving_decode_tok_per_s", "value": r1(rec["decode_tok_per_s"]), "unit": "tokens/s",
                    "n_gpus": world, "steps": rec["requests"], "warmup": 0, "higher_is_better": True, "scaling": "weak",
                    "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": args.impl,
                    "ttft_p50_ms": r1(rec["ttft_p50_ms"]), "ttft_p99_ms": r1(rec["ttft_p99_ms"]),
                    "offline_tok_per_s": r1(rec["offline_tok_per_s"]), "output_tokens": rec["output_tokens"],
                    "wall_s": round(rec["wall_s"], 2), "config": serving_config(), "engine": rec["engine"], "clocks": clk,
                    "e2e": {"value": r1(rec["decode_tok_per_s"]), "unit": "tokens/s",
                            "note": "prompts are host token lists copied to the device per prefill; every sampled token is "
                                    "read back to the host each decode step"},
                    "gpu_launches": rec["launches"],
                    "timing": "wall clock around the trace with a device synchronisation on both sides (arrival-driven "
                              "workload); max over replicas"}))
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()
        return 0
    if args.impl == "reference":
        try:
            res, why = run_reference(args, cfg, rank, local_rank, world)
        except torch.cuda.OutOfMemoryError as e:
            res, why = None, f"reference ran out of device memory on this config: {str(e)[:120]}"
        if res is None:
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": why}))
            return 0
    else:
        gave_up = None
        try:
            res = run_native(args, cfg, rank, local_rank, world)
        except PeerPathGaveUp as e:
            gave_up = str(e)        # leave the handler first: the traceback keeps the first model alive
        if gave_up is not None:
            import gc
            gc.collect()
            torch.cuda.empty_cache()
            args.comm, args.fused_optimizer = "torch", "off"
            res = run_native(args, cfg, rank, local_rank, world)
            res["comm"] += f" (the peer-memory collectives gave up in the first step and the run was repeated: {gave_up})"
    # second half of the headline metric, short form: a serving replica per GPU after the training model is gone
    n_serv = 160 if args.serving_requests is None else args.serving_requests
    serving = None
    if n_serv > 0 and args.config == "fsdp_1p3b":
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        try:
            rec = run_serving(args, rank, local_rank, world, n_serv)
        except Exception as e:      # the training numbers above stand whatever happens to the serving record
            rec = {"unavailable": f"{type(e).__name__}: {str(e)[:160]}"}
        serving = gather_serving(rec, world)
    if rank == 0:
        ms_step = res["ms"] / args.steps
        value = res["tokens_per_step"] / (ms_step / 1e3)
        e2e = res["tokens_per_step"] / (res["ms_e2e"] / args.steps / 1e3)
        line = {
            "metric": "train_tokens_per_s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": args.impl,
            "config": {"model": cfg["model"], "global_batch": cfg["micro_batch"] * world, "seq_len": cfg["context_length"],
                       "parallelism": res["parallelism"], "micro_batch_per_gpu": cfg["micro_batch"],
                       "vocab": cfg["vocab_size"], "d_model": cfg["d_model"], "layers": cfg["num_layers"],
                       "heads": cfg["num_heads"], "d_ff": cfg["d_ff"], "l2_policy": l2_policy(cfg)},
            "optimizer": res["optimizer"], "comm": res["comm"], "comm_launches_timed_region": res["comm_launches"],
            "activation_checkpointing": res["activation_checkpointing"],
            "clocks": res["clocks"],
            "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "ms_per_step": round(res["ms_e2e"] / args.steps, 3),
                    "h2d_bytes_per_step": res["h2d"], "d2h_bytes_per_step": res["d2h"]},
            "gpu_launches": res["launches"],
            "final_loss": round(res["loss"], 4), "peak_mem_gb": round(res["mem_gb"], 2),
        }
        if serving is not None:
            if "unavailable" not in serving:
                serving = {k: (round(v, 1) if isinstance(v, float) else v) for k, v in serving.items()}
                serving["metric"] = "serving_decode_tok_per_s"
                serving["config"] = serving_config()
            line["serving"] = serving
        print(json.dumps(line))
    if world > 1 or args.impl == "reference":
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
