"""YAML run configuration with the reference's schema (configures/sample.yaml:1-30, train.py:92-109).

Required sections and keys are those the reference indexes without defaults: ``model``,
``training``, ``optimizer``, ``dataset``.  Extra keys the reference lacks are optional here and get
defaults: ``training.seed``, ``training.dtype``, ``training.activation_checkpointing``,
``training.resume``, ``training.step_timeout_s``, ``optimizer.betas``, ``optimizer.eps``, ``fsdp.comm``,
``fsdp.fused_optimizer``, ``ddp.bucket_size_mb``, and a whole optional ``serving`` section.
"""
from __future__ import annotations

import yaml

REQUIRED = {
    "model": ["vocab_size", "context_length", "d_model", "num_layers", "num_heads", "d_ff", "rope_theta"],
    "training": ["device", "batch_size", "max_steps", "val_interval", "gpu_log_interval", "checkpoint_dir", "wandb",
                 "wandb_project"],
    "optimizer": ["learning_rate_max", "learning_rate_min", "weight_decay", "max_grad_norm", "warmup_steps",
                  "decay_steps"],
    "dataset": ["train_path", "val_path"],
}

DEFAULTS = {
    "training": {"seed": None, "dtype": "bf16", "activation_checkpointing": False, "resume": None,
                 "val_last_position_only": True, "metrics_file": None, "step_timeout_s": 600.0},
    "optimizer": {"betas": [0.9, 0.95], "eps": 1e-8},
    # fused_optimizer: "off" = reduce-scatter, exact global-norm clip, one AdamW launch; "delayed_clip" = AdamW inside
    # each unit's reduce-scatter, clipping with the coefficient of the previous step's gradient norm
    "fsdp": {"comm": "auto", "fused_optimizer": "off"},
    "ddp": {"bucket_size_mb": 25.0, "comm": "auto"},
    "serving": {"page_size": 16, "max_batch": 64, "max_context": 2560, "num_pages": 0, "arrival_rate": 20.0,
                "num_requests": 1024, "prompt_len": [128, 2048], "output_len": [64, 512], "seed": 0},
}


def load_config(path: str) -> dict:
    with open(path, "r") as f:
        return yaml.safe_load(f)


def validate(cfg: dict, world_size: int = 1, require_dataset: bool = True) -> dict:
    """Check required keys, fill optional ones, coerce numeric strings such as ``6.0e-4``."""
    out = {k: dict(v) if isinstance(v, dict) else v for k, v in cfg.items()}
    for section, keys in REQUIRED.items():
        if section == "dataset" and not require_dataset:
            continue
        if section not in out:
            raise KeyError(f"config section '{section}' is missing")
        for k in keys:
            if k not in out[section]:
                raise KeyError(f"config key '{section}.{k}' is missing")
    for section, defaults in DEFAULTS.items():
        sec = out.setdefault(section, {})
        for k, v in defaults.items():
            sec.setdefault(k, v)
    o = out["optimizer"]
    for k in ("learning_rate_max", "learning_rate_min", "weight_decay", "max_grad_norm", "eps"):
        o[k] = float(o[k])
    bs = out["training"]["batch_size"]
    if world_size > 1 and bs % world_size:
        raise ValueError(f"training.batch_size ({bs}) must be divisible by the world size ({world_size}); "
                         "the reference silently floors it")
    if out["fsdp"]["fused_optimizer"] not in ("off", "delayed_clip"):
        raise ValueError("fsdp.fused_optimizer must be 'off' or 'delayed_clip'")
    m = out["model"]
    if m["d_model"] % m["num_heads"]:
        raise ValueError("model.d_model must be divisible by model.num_heads")
    return out
