"""Checkpoints: the reference's single-file format plus sharded optimizer state for FSDP.

Single file (reference: train.py:23-52): ``torch.save({"model": state_dict, "iteration": int
[, "optimizer": optimizer.state_dict()]})`` next to a ``model_config.json`` holding the model's
constructor arguments.  Files written here load in the reference and vice versa; either FFN key
layout is accepted on load.

Sharded (new; the reference saves no optimizer state under FSDP and cannot resume): every rank
writes ``shard_{rank:05d}.pt`` with its slices of master weights, m and v; rank 0 writes
``manifest.json``.  Loading re-slices, so a run may resume on a different world size.
"""
from __future__ import annotations

import json
import os

import torch


def save_checkpoint(model, optimizer, iteration: int, path, save_optimizer: bool = True, state_dict=None) -> None:
    """Write ``path`` (and ``model_config.json`` beside it) in the reference format."""
    ckpt = {"model": state_dict if state_dict is not None else model.state_dict(), "iteration": iteration}
    if save_optimizer and optimizer is not None:
        ckpt["optimizer"] = optimizer.state_dict()
    parent = os.path.dirname(path)
    if parent:
        os.makedirs(parent, exist_ok=True)
    tmp = f"{path}.tmp"
    torch.save(ckpt, tmp)
    os.replace(tmp, path)
    with open(os.path.join(parent, "model_config.json"), "w") as f:
        json.dump(model.config, f)


def load_checkpoint(path, model, optimizer=None) -> int:
    ckpt = torch.load(path, map_location="cpu")
    model.load_state_dict(ckpt["model"])
    if optimizer is not None and "optimizer" in ckpt:
        sd = ckpt["optimizer"]
        for st in sd.get("state", {}).values():     # accept both step-count conventions (t = steps or steps + 1)
            if "t" in st and st["t"] < 1:
                st["t"] = 1
        optimizer.load_state_dict(sd)
    return int(ckpt["iteration"])


# ------------------------------------------------------------------------------ sharded
def save_sharded(fsdp, optimizer, iteration: int, directory: str) -> None:
    """Collective: every rank writes its own shard file; rank 0 also writes the manifest."""
    os.makedirs(directory, exist_ok=True)
    sa = fsdp.shard_arena
    flat = getattr(optimizer, "_flat", {}).get(0) if optimizer is not None else None
    payload = {"iteration": iteration, "rank": fsdp.rank, "world_size": fsdp.world_size,
               "units": [{"name": u.name, "original_numel": u.original_numel, "shard_numel": u.shard_numel}
                         for u in fsdp.fsdp_units],
               "master": sa.master.detach().cpu()}
    if flat is not None:
        payload.update(m=flat["m"].cpu(), v=flat["v"].cpu(), t=int(flat["t"]))
    tmp = os.path.join(directory, f"shard_{fsdp.rank:05d}.pt.tmp")
    torch.save(payload, tmp)
    os.replace(tmp, tmp[:-4])
    if fsdp.rank == 0:
        with open(os.path.join(directory, "manifest.json"), "w") as f:
            json.dump({"iteration": iteration, "world_size": fsdp.world_size, "model_config": fsdp.module.config,
                       "units": payload["units"]}, f)
    fsdp.comm.barrier()


def _unit_full(shards: list[dict], key: str, name: str) -> torch.Tensor:
    """Concatenate the slices of the unit called ``name`` from every saved rank and drop the padding."""
    names = [u["name"] for u in shards[0]["units"]]
    if name not in names:
        raise KeyError(f"sharded checkpoint has no unit {name!r} (it holds {names})")
    unit_idx = names.index(name)
    parts = []
    for sh in shards:
        off = sum(u["shard_numel"] for u in sh["units"][:unit_idx])
        n = sh["units"][unit_idx]["shard_numel"]
        parts.append(sh[key][off:off + n])
    return torch.cat(parts)[:shards[0]["units"][unit_idx]["original_numel"]]


def load_sharded(fsdp, optimizer, directory: str) -> int:
    """Resume from ``save_sharded`` output, re-slicing for the current world size."""
    with open(os.path.join(directory, "manifest.json")) as f:
        manifest = json.load(f)
    shards = [torch.load(os.path.join(directory, f"shard_{r:05d}.pt"), map_location="cpu")
              for r in range(manifest["world_size"])]
    sa = fsdp.shard_arena
    has_opt = optimizer is not None and "m" in shards[0]
    if has_opt:
        st = {"t": shards[0]["t"], "m": torch.zeros_like(sa.master), "v": torch.zeros_like(sa.master)}
    for ui, (u, seg) in enumerate(zip(fsdp.fsdp_units, sa.segments)):
        lo = fsdp.rank * u.shard_numel
        for key, dst in (("master", sa.master),) + ((("m", st["m"]), ("v", st["v"])) if has_opt else ()):
            full = _unit_full(shards, key, u.name)
            piece = full[lo:lo + u.shard_numel]
            d = dst[seg.start:seg.start + seg.numel]
            d.zero_()
            d[:piece.numel()].copy_(piece)
    sa._mirror_fresh = False
    if has_opt:
        optimizer._flat[0] = st
    return int(manifest["iteration"])
