"""train.py / generate.py end to end on CPU with a tiny model (single process, resume, generation)."""
import json
import os
import sys

import numpy as np
import pytest
import torch
import yaml

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DATA = os.path.join(os.path.dirname(__file__), "data")


def _config(tmp_path, max_steps=6):
    rng = np.random.default_rng(0)
    for name in ("train", "val"):
        rng.integers(0, 300, size=4096, dtype=np.uint32).tofile(tmp_path / f"{name}.bin")
    cfg = {
        "model": dict(vocab_size=300, context_length=32, d_model=64, num_layers=2, num_heads=4, d_ff=136, rope_theta=10000.0),
        "training": dict(device="cpu", batch_size=4, max_steps=max_steps, val_interval=3, gpu_log_interval=100,
                         checkpoint_dir=str(tmp_path / "ckpt"), wandb=False, wandb_project="x", seed=0,
                         metrics_file=str(tmp_path / "metrics.jsonl")),
        "optimizer": dict(learning_rate_max="1.0e-2", learning_rate_min="1.0e-3", weight_decay=0.1, max_grad_norm=1.0,
                          warmup_steps=2, decay_steps=6),
        "dataset": dict(train_path=str(tmp_path / "train.bin"), val_path=str(tmp_path / "val.bin")),
    }
    path = tmp_path / "cfg.yaml"
    path.write_text(yaml.safe_dump(cfg))
    return str(path)


@pytest.mark.parametrize("native", [False, True])
def test_train_resume_generate(tmp_path, native, capsys):
    sys.path.insert(0, ROOT)
    import generate
    import train
    cfg = _config(tmp_path)
    train.train_worker(0, 1, [], cfg, False, False, False, native)
    out = capsys.readouterr().out
    assert "[Rank 0] Step 5: loss = " in out and "tok/s = " in out and "[Validation] Step 3" in out
    ck = tmp_path / "ckpt"
    assert (ck / "ckpt_3.pt").exists() and (ck / "ckpt_final.pt").exists() and (ck / "model_config.json").exists()
    final = torch.load(ck / "ckpt_final.pt")
    assert final["iteration"] == 6 and "optimizer" in final
    assert json.load(open(ck / "model_config.json"))["use_custom_triton"] is native
    lines = [json.loads(l) for l in open(tmp_path / "metrics.jsonl")]
    assert sum("train/loss" in r for r in lines) == 6
    # resume from the step-3 checkpoint: continues at step 3 and ends with the same iteration count
    train.train_worker(0, 1, [], cfg, False, False, False, native, resume=str(ck / "ckpt_3.pt"))
    out = capsys.readouterr().out
    assert "resumed from" in out and "Step 3:" in out and "Step 2:" not in out
    # generation from the final checkpoint with the golden tokenizer files
    generate.main(["--config", str(ck / "model_config.json"), "--checkpoint", str(ck / "ckpt_final.pt"),
                   "--vocab", os.path.join(DATA, "vocab.json"), "--merges", os.path.join(DATA, "merges.json"),
                   "--max-tokens", "5", "--temperature", "0", "--device", "cpu", "--prompt", "the "])
    assert isinstance(capsys.readouterr().out, str)


def test_config_validation_rejects_indivisible_batch(tmp_path):
    from llm_systems_from_scratch_b200.utils.config import load_config, validate
    cfg = load_config(_config(tmp_path))
    with pytest.raises(ValueError):
        validate(cfg, world_size=3)
    del cfg["optimizer"]["warmup_steps"]
    with pytest.raises(KeyError):
        validate(cfg)
    for name in ("sample", "cpu_tiny", "ddp_124m", "fsdp_1p3b", "fsdp_7b", "serve_1p3b"):
        validate(load_config(os.path.join(ROOT, "configures", f"{name}.yaml")), world_size=8)


def test_profile_flag_writes_chrome_trace(tmp_path, monkeypatch):
    """B200_PROFILE_STEPS (set by --profile N) wraps N steps in torch.profiler and writes a trace per rank."""
    sys.path.insert(0, ROOT)
    import train
    cfg = _config(tmp_path, max_steps=7)
    monkeypatch.setenv("B200_PROFILE_STEPS", "2")
    train.train_worker(0, 1, [], cfg, False, False, False, True)
    trace = tmp_path / "ckpt" / "trace_rank0.json"
    assert trace.exists() and trace.stat().st_size > 1000


def test_bench_reference_arm_without_a_gpu_says_so_and_exits_zero():
    """``bench.py --impl reference`` must never fail the caller: without a CUDA device it prints its one-line
    ``unavailable`` record and exits 0; the default arm needs a GPU and says so by raising."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    ref = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference"], capture_output=True,
                         text=True, env=env, timeout=300)
    assert ref.returncode == 0, ref.stderr[-400:]
    rec = json.loads(ref.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and "unavailable" in rec
    own = subprocess.run([sys.executable, os.path.join(root, "bench.py")], capture_output=True, text=True, env=env,
                         timeout=300)
    assert own.returncode != 0 and "no CUDA device" in own.stderr


@pytest.mark.parametrize("parallel", ["ddp", "fsdp"])
def test_launcher_restarts_from_the_newest_checkpoint_after_a_rank_failure(tmp_path, parallel):
    """Recovery is restart-from-checkpoint: with ``--max-restarts 1`` a run in which one of two gloo ranks raises
    before step 4 (a failure made on the host, nothing in flight) starts again from the step-3 checkpoint - a single
    file under DDP, a sharded directory under FSDP - and runs to the end; without restarts left the failure surfaces."""
    import subprocess
    cfg = _config(tmp_path, max_steps=8)
    env = dict(os.environ, B200_INJECT_FAIL_STEP="4:1", MASTER_ADDR="127.0.0.1", CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, os.path.join(ROOT, "train.py"), "--config", cfg, "--parallel", parallel, "--world-size", "2"]
    run = subprocess.run(cmd + ["--max-restarts", "1"], capture_output=True, text=True, env=env, timeout=600)
    assert run.returncode == 0, run.stderr[-800:]
    newest = "sharded_3" if parallel == "fsdp" else "ckpt_3.pt"
    assert f"restart 1/1 from {tmp_path / 'ckpt' / newest}" in run.stdout
    assert "resumed from" in run.stdout and "Step 7:" in run.stdout
    assert (tmp_path / "ckpt" / "ckpt_final.pt").exists()
    # the same failure with no restart allowed ends the job with the worker's error
    import shutil
    shutil.rmtree(tmp_path / "ckpt")
    run = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert run.returncode != 0 and "failure injected on the host" in run.stderr


def test_latest_checkpoint_picks_the_highest_step(tmp_path):
    sys.path.insert(0, ROOT)
    import train
    assert train.latest_checkpoint(str(tmp_path / "missing")) is None
    d = tmp_path / "ck"
    d.mkdir()
    assert train.latest_checkpoint(str(d)) is None
    for name in ("ckpt_3.pt", "ckpt_12.pt", "ckpt_final.pt", "model_config.json"):
        (d / name).write_text("x")
    assert train.latest_checkpoint(str(d)).endswith("ckpt_12.pt")
    (d / "sharded_20").mkdir()
    (d / "sharded_final").mkdir()
    (d / "sharded_30").write_text("not a directory")
    assert train.latest_checkpoint(str(d)).endswith("sharded_20")


def test_train_under_an_external_launcher(tmp_path):
    """``python -m torch.distributed.run ... train.py --parallel fsdp``: every process is one rank (rank, world size
    and rendezvous from the environment) instead of train.py spawning the ranks itself."""
    import socket
    import subprocess
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    cfg = _config(tmp_path, max_steps=5)
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    run = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "train.py"),
                          "--config", cfg, "--parallel", "fsdp"], capture_output=True, text=True, env=env, timeout=600)
    assert run.returncode == 0, run.stderr[-800:]
    assert "[Rank 0] Step 4:" in run.stdout and "[Rank 1] Step 4:" in run.stdout
    assert (tmp_path / "ckpt" / "sharded_final").is_dir()
