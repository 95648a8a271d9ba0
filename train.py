#!/usr/bin/env python
"""Training driver: YAML config + flags -> single-process, DDP or FSDP training.

Command line and behaviour follow the reference driver (train.py:75-353):

    python train.py --config configures/sample.yaml [--amp] [--compile] [--flash-attn]
                    [--custom-triton] [--parallel ddp|fsdp] [--world-size N] [--resume PATH]

On a CUDA device the hand-written sm_100a kernel path (fused engine, fused AdamW, fused chunked loss)
is the default; ``--eager`` selects the plain PyTorch modules instead (the oracle the kernels are tested
against).  ``--custom-triton`` is accepted so that the reference's command lines keep working; on CPU it
selects the same fused engine running on its fp32 PyTorch statement.  Distributed runs spawn one
process per GPU and rendezvous on 127.0.0.1.  YAML ``batch_size`` is global; each rank takes
``batch_size // world_size`` (validated to divide evenly).  Checkpoints use the reference's
single-file format; FSDP additionally writes sharded optimizer state so that runs can resume.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from llm_systems_from_scratch_b200.data.loader import sample_batch  # noqa: E402
from llm_systems_from_scratch_b200.models.transformer import TransformerLM  # noqa: E402
from llm_systems_from_scratch_b200.ops.functional import clip_gradient, cross_entropy  # noqa: E402
from llm_systems_from_scratch_b200.optim.adamw import AdamW, FusedAdamW, cosine_lr_schedule  # noqa: E402
from llm_systems_from_scratch_b200.utils import checkpoint as ckpt_io  # noqa: E402
from llm_systems_from_scratch_b200.utils.config import load_config, validate  # noqa: E402
from llm_systems_from_scratch_b200.utils.metrics import MetricsLogger, StepTimer, get_gpu_stats, nvtx_range  # noqa: E402,F401
from llm_systems_from_scratch_b200.utils.watchdog import Heartbeat, StepWatchdog  # noqa: E402


def save_checkpoint(model, optimizer, iteration: int, path, save_optimizer: bool = True) -> None:
    ckpt_io.save_checkpoint(model, optimizer, iteration, path, save_optimizer)


def load_checkpoint(path, model, optimizer) -> int:
    return ckpt_io.load_checkpoint(path, model, optimizer)


def detect_device() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


def _init_wandb(train_cfg, model_cfg, batch_size, lr_max, parallel, world_size):
    try:
        import wandb
    except ImportError:
        print("wandb requested but not importable; continuing without it")
        return None
    name = f"bs{batch_size}_lr{lr_max}_layer{model_cfg['num_layers']}"
    if parallel:
        name += f"_{'+'.join(parallel)}_ws{world_size}"
    try:
        return wandb.init(project=train_cfg["wandb_project"], name=name,
                          config={"batch_size": batch_size, "learning_rate": lr_max,
                                  "context_length": model_cfg["context_length"], "d_model": model_cfg["d_model"],
                                  "max_steps": train_cfg["max_steps"], "parallel": parallel, "world_size": world_size})
    except Exception as e:  # no network on the training box is normal
        print(f"wandb.init failed ({e}); continuing without it")
        return None


def train_worker(rank: int = 0, world_size: int = 1, parallel: list[str] | None = None,
                 config_path: str = "./configures/sample.yaml", use_amp: bool = False, use_compile: bool = False,
                 use_flash_attn: bool = False, use_custom_triton: bool = False, resume: str | None = None,
                 backend: str | None = None, eager: bool = False):
    parallel = parallel or []
    distributed = len(parallel) > 0
    use_fsdp, use_ddp = "fsdp" in parallel, "ddp" in parallel
    torch.set_float32_matmul_precision("high")
    cfg = validate(load_config(config_path), world_size if distributed else 1)
    model_cfg, train_cfg, optim_cfg, data_cfg = cfg["model"], cfg["training"], cfg["optimizer"], cfg["dataset"]
    batch_size, max_steps = train_cfg["batch_size"], train_cfg["max_steps"]
    val_interval, gpu_log_interval = train_cfg["val_interval"], train_cfg["gpu_log_interval"]
    checkpoint_dir, context_length = train_cfg["checkpoint_dir"], model_cfg["context_length"]
    lr_max, lr_min = optim_cfg["learning_rate_max"], optim_cfg["learning_rate_min"]
    max_grad_norm = optim_cfg["max_grad_norm"]
    resume = resume or train_cfg.get("resume")

    heartbeat = None
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        use_cuda = torch.cuda.is_available() and train_cfg["device"] != "cpu"
        backend = backend or ("nccl" if use_cuda else "gloo")
        dist.init_process_group(backend, rank=rank, world_size=world_size)
        if use_cuda:
            local_rank = int(os.environ.get("LOCAL_RANK", rank % torch.cuda.device_count()))
            torch.cuda.set_device(local_rank)
            device = f"cuda:{local_rank}"
        else:
            device = "cpu"
        store = dist.distributed_c10d._get_default_store()
        heartbeat = Heartbeat(store, rank, world_size, interval=1.0, timeout=60.0).start()
    else:
        device = detect_device() if train_cfg["device"] == "auto" else train_cfg["device"]
    amp_device_type = device.split(":")[0]
    if amp_device_type == "cuda" and not eager:
        use_custom_triton = True        # the kernels of this package are the default path on a GPU
    if train_cfg.get("seed") is not None:
        torch.manual_seed(int(train_cfg["seed"]) + rank)

    wandb_run = None
    if train_cfg["wandb"] and rank == 0:
        wandb_run = _init_wandb(train_cfg, model_cfg, batch_size, lr_max, parallel, world_size)
    logger = MetricsLogger(rank, train_cfg.get("metrics_file"), wandb_run)
    print(f"[Rank {rank}] device: {device}")

    train_data = np.memmap(data_cfg["train_path"], dtype=np.uint32, mode="r")
    val_data = np.memmap(data_cfg["val_path"], dtype=np.uint32, mode="r")

    mkeys = ("d_model", "num_heads", "d_ff", "vocab_size", "context_length", "num_layers", "rope_theta")
    model = TransformerLM(**{k: model_cfg[k] for k in mkeys}, use_flash_attn=use_flash_attn,
                          use_custom_triton=use_custom_triton).to(device)
    model.activation_checkpointing = bool(train_cfg.get("activation_checkpointing"))
    inner_model = model
    native = use_fsdp or model.native_supported()
    if use_compile and not native:
        model = torch.compile(model)
    if use_fsdp:
        from llm_systems_from_scratch_b200.parallel.fsdp import FSDP
        model = FSDP(model, comm=cfg["fsdp"]["comm"])
    elif use_ddp:
        from llm_systems_from_scratch_b200.parallel.ddp import DDP
        model = DDP(model, bucket_size_mb=cfg["ddp"]["bucket_size_mb"], comm=cfg["ddp"]["comm"])
    model.train()

    opt_cls = FusedAdamW if (use_custom_triton or use_fsdp) else AdamW
    optimizer = opt_cls(params=model.parameters(), lr=lr_max, weight_decay=optim_cfg["weight_decay"],
                        betas=tuple(optim_cfg["betas"]), eps=optim_cfg["eps"])
    # AdamW inside each unit's reduce-scatter (clips with the previous step's coefficient): fsdp.fused_optimizer
    fused_opt = (use_fsdp and cfg["fsdp"]["fused_optimizer"] == "delayed_clip"
                 and model.attach_optimizer(optimizer, max_grad_norm))
    if use_fsdp:
        print(f"[Rank {rank}] fsdp: comm={type(model.comm).__name__} fused_optimizer="
              f"{'delayed_clip' if fused_opt else 'off'}")
    on_gpu = amp_device_type == "cuda"
    if on_gpu:
        from llm_systems_from_scratch_b200.ops import native as native_ops
    # A step that takes longer than training.step_timeout_s (a stuck collective, a hung peer) is reported from the
    # watchdog thread; the loop raises at the next step boundary.
    watchdog = StepWatchdog(float(train_cfg["step_timeout_s"]),
                            on_timeout=lambda: print(f"[Rank {rank}] step watchdog: step exceeded "
                                                     f"{train_cfg['step_timeout_s']} s", flush=True))

    def rejoin():
        """After host work that only some ranks do (rank 0 writing a checkpoint): meet on the host before any device
        collective resumes, so that the bounded device waits never see the skew."""
        if distributed:
            dist.barrier()

    start_step = 0
    if resume:
        if use_fsdp and os.path.isdir(resume):
            start_step = ckpt_io.load_sharded(model, optimizer, resume)
        elif use_fsdp:
            state = torch.load(resume, map_location="cpu")
            model.load_full_state_dict(state["model"])
            start_step = int(state["iteration"])
        else:
            start_step = load_checkpoint(resume, inner_model, optimizer)
        print(f"[Rank {rank}] resumed from {resume} at step {start_step}")

    local_batch = batch_size // world_size if distributed else batch_size
    timer = StepTimer(device)

    def loss_of(x, y):
        if native:
            return model.loss(x, y)     # fused head: logits are never materialised
        with torch.autocast(device_type=amp_device_type, dtype=torch.bfloat16, enabled=use_amp):
            logits = model(x)
            return cross_entropy(logits.view(-1, logits.size(-1)).float(), y.view(-1))

    # optional torch.profiler trace of a few steps (B200_PROFILE_STEPS=N, set by --profile N): Chrome trace per rank
    profile_steps = int(os.environ.get("B200_PROFILE_STEPS", "0"))
    profiler = None
    inject = os.environ.get("B200_INJECT_FAIL_STEP")      # host-made failure for the restart tests: "<step>[:<rank>]"
    for step in range(start_step, max_steps):
        if heartbeat is not None:
            heartbeat.check()          # between steps: nothing of this rank is in flight
        if inject and resume is None:
            at, _, who = inject.partition(":")
            if step == int(at) and rank == int(who or 0):
                raise RuntimeError(f"rank {rank}: failure injected on the host before step {step}")
        if watchdog.expired:
            raise RuntimeError(f"step {step - 1} exceeded training.step_timeout_s; restart from the last checkpoint")
        watchdog.arm()
        if profile_steps and step == start_step + 3:
            from torch.profiler import ProfilerActivity, profile
            acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
            profiler = profile(activities=acts)
            profiler.__enter__()
        if profiler is not None and step == start_step + 3 + profile_steps:
            profiler.__exit__(None, None, None)
            os.makedirs(checkpoint_dir, exist_ok=True)
            profiler.export_chrome_trace(os.path.join(checkpoint_dir, f"trace_rank{rank}.json"))
            profiler = None
        timer.start()
        lr = cosine_lr_schedule(step, lr_max, lr_min, optim_cfg["warmup_steps"], optim_cfg["decay_steps"])
        for group in optimizer.param_groups:
            group["lr"] = lr
        with nvtx_range("data"):
            x, y = sample_batch(train_data, local_batch, context_length, device)
        model.zero_grad()
        with nvtx_range("forward"):
            loss = loss_of(x, y)
        with nvtx_range("backward"):
            loss.backward()
            if distributed:
                model.finish_gradient_synchronization()
        with nvtx_range("optimizer"):
            if fused_opt:
                model.finish_fused_step()      # the update ran inside the reduce-scatters; this norm clips the next step
            else:
                clip_gradient(model.parameters(), max_grad_norm)
            optimizer.step()
        loss_value = loss.item()
        if on_gpu:
            # the loss read-back has synchronised the device: a bounded device wait that gave up during this step
            # (a peer more than the limit late) left its collective undone - stop here rather than train on
            native_ops.check_status()
        watchdog.disarm()
        step_time = timer.stop()
        logger.step_line(step, loss_value, lr, step_time, batch_size * context_length / step_time)
        logger.log({"train/loss": loss_value, "train/lr": lr, "step": step, "step_time_s": step_time})

        if step % val_interval == 0 and step > 0:
            model.eval()
            with torch.no_grad():
                xv, yv = sample_batch(val_data, local_batch, context_length, device)
                if train_cfg.get("val_last_position_only", True):
                    logits = model(xv)
                    val_loss = cross_entropy(logits[:, -1, :].float(), yv[:, -1])
                else:
                    val_loss = loss_of(xv, yv)
                print(f"[Rank {rank}] [Validation] Step {step}: val_loss = {val_loss.item():.4f}")
                logger.log({"val/loss": val_loss.item(), "step": step})
            model.train()
            if use_fsdp:
                ckpt_io.save_sharded(model, optimizer, step, os.path.join(checkpoint_dir, f"sharded_{step}"))
            elif not distributed or rank == 0:
                save_checkpoint(inner_model, optimizer, step, os.path.join(checkpoint_dir, f"ckpt_{step}.pt"))
            rejoin()
            if on_gpu:
                native_ops.check_status()
                guards = getattr(getattr(model, "comm", None), "check_guards", None)
                if guards is not None:
                    guards()        # canary bands around the peer-addressable buffers are intact

        if wandb_run is not None and step % gpu_log_interval == 0 and torch.cuda.is_available():
            rec = {"allocated_memory": int(torch.cuda.memory_allocated() / 1024 ** 2),
                   "cached_memory": int(torch.cuda.memory_reserved() / 1024 ** 2)}
            for idx, stat in enumerate(get_gpu_stats()):
                util, mem, temp = map(float, stat)
                rec.update({f"gpu_{idx}_utilization": util, f"gpu_{idx}_memory_used": mem, f"gpu_{idx}_temperature": temp})
            logger.log(rec)

    final = os.path.join(checkpoint_dir, "ckpt_final.pt")
    if use_fsdp:
        state = model.full_state_dict()            # collective on every rank
        ckpt_io.save_sharded(model, optimizer, max_steps, os.path.join(checkpoint_dir, "sharded_final"))
        if rank == 0:
            ckpt_io.save_checkpoint(inner_model, None, max_steps, final, save_optimizer=False, state_dict=state)
    elif not distributed or rank == 0:
        save_checkpoint(inner_model, optimizer, max_steps, final)
    logger.close()
    watchdog.stop()
    if heartbeat is not None:
        heartbeat.mark_done()
        heartbeat.stop()
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=str, default="./configures/sample.yaml", help="Path to training config YAML")
    ap.add_argument("--amp", action="store_true", help="bf16 autocast on the eager path")
    ap.add_argument("--compile", action="store_true", help="torch.compile the eager model (ignored on the native path)")
    ap.add_argument("--flash-attn", action="store_true", help="fused attention on the eager path")
    ap.add_argument("--custom-triton", "--native", dest="custom_triton", action="store_true",
                    help="run the fused engine (the default on a CUDA device; on CPU its fp32 PyTorch statement)")
    ap.add_argument("--eager", action="store_true",
                    help="plain PyTorch modules on the GPU instead of this package's kernels (the test oracle)")
    ap.add_argument("--parallel", nargs="+", default=[], choices=["ddp", "fsdp"])
    ap.add_argument("--world-size", type=int, default=2)
    ap.add_argument("--resume", type=str, default=None, help="checkpoint file or sharded checkpoint directory")
    ap.add_argument("--profile", type=int, default=0, metavar="N",
                    help="torch.profiler Chrome trace of N steps (after 3 warm-up steps) into the checkpoint directory")
    ap.add_argument("--nvtx", action="store_true", help="NVTX ranges per block, phase and collective")
    ap.add_argument("--max-restarts", type=int, default=0, metavar="N",
                    help="after a failed run (a worker that died, a rank failure, a kernel status error) start again "
                         "from the newest periodic checkpoint, at most N times")
    args = ap.parse_args()
    if args.profile:
        os.environ["B200_PROFILE_STEPS"] = str(args.profile)   # inherited by spawned ranks
    if args.nvtx:
        os.environ["B200_NVTX"] = "1"
    if "ddp" in args.parallel and "fsdp" in args.parallel:
        raise ValueError("--parallel ddp and fsdp are mutually exclusive (both are data parallelism)")
    if "fsdp" in args.parallel and args.compile:
        raise ValueError("--parallel fsdp and --compile are not compatible: FSDP always runs the fused engine")
    if args.eager and ("fsdp" in args.parallel or args.custom_triton):
        raise ValueError("--eager excludes --custom-triton and --parallel fsdp (FSDP always runs the fused engine)")
    if args.parallel and "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        # started by an external launcher (python -m torch.distributed.run ... train.py --parallel ...): this process
        # is one rank; rendezvous, rank and world size come from the environment and --world-size is ignored
        train_worker(int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), args.parallel, args.config, args.amp,
                     args.compile, args.flash_attn, args.custom_triton, args.resume, None, args.eager)
        return
    if args.parallel:
        mp.set_start_method("spawn", force=True)
    resume, restarts = args.resume, 0
    while True:
        common = (args.config, args.amp, args.compile, args.flash_attn, args.custom_triton, resume, None, args.eager)
        try:
            if args.parallel:
                mp.spawn(train_worker, args=(args.world_size, args.parallel, *common), nprocs=args.world_size,
                         join=True)
            else:
                train_worker(0, 1, [], *common)
            return
        except KeyboardInterrupt:
            raise
        except Exception as e:      # noqa: BLE001 - a worker died (mp.spawn re-raises it), a rank failure, a kernel error
            if restarts >= args.max_restarts:
                raise
            restarts += 1
            newest = latest_checkpoint(load_config(args.config)["training"]["checkpoint_dir"])
            resume = newest or resume
            print(f"[launcher] run failed ({type(e).__name__}: {str(e).strip().splitlines()[-1][:160] if str(e).strip() else ''}); "
                  f"restart {restarts}/{args.max_restarts} from {resume or 'the beginning'}", flush=True)


def latest_checkpoint(checkpoint_dir: str) -> str | None:
    """The newest periodic checkpoint of a run: ``sharded_<step>`` directories (FSDP, any world size can load them) or
    ``ckpt_<step>.pt`` files; None if there is none yet."""
    best, best_step = None, -1
    if not os.path.isdir(checkpoint_dir):
        return None
    for name in os.listdir(checkpoint_dir):
        stem = name[:-3] if name.endswith(".pt") else name
        kind, _, num = stem.rpartition("_")
        if kind in ("sharded", "ckpt") and num.isdigit() and int(num) > best_step:
            if kind == "sharded" and not os.path.isdir(os.path.join(checkpoint_dir, name)):
                continue
            best, best_step = os.path.join(checkpoint_dir, name), int(num)
    return best


if __name__ == "__main__":
    main()
