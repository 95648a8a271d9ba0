#!/usr/bin/env python
"""Serving benchmark / driver: replays a Poisson request trace through the continuous-batching engine.

    python serve.py --config configures/serve_1p3b.yaml [--num-requests N] [--rate R] [--offline]
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 serve.py ...   (one replica per GPU)
    python serve.py --config configures/serve_1p3b.yaml --checkpoint ckpt_final.pt --http 8000   (online: POST /generate)

Weights are random-init unless ``--checkpoint`` points at a checkpoint written by train.py.  Each replica
serves its own trace (seed + rank); rank 0 prints one JSON line with the aggregate decode tokens/s and
the time-to-first-token percentiles.  ``--impl reference`` replays the head of the same trace through
the reference-style loop (one request at a time, greedy argmax over a full re-forward, no KV cache).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def naive_loop(model, requests, device, limit_s: float):
    """Per-request greedy loop without a KV cache (what the reference's generate() does), for a baseline."""
    t0 = time.perf_counter()
    out_tokens, ttft, served = 0, [], 0
    for r in requests:
        now = time.perf_counter() - t0
        if now < r.arrival:
            time.sleep(r.arrival - now)
        ids = torch.tensor([r.prompt], device=device)
        for k in range(r.max_new_tokens):
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16, enabled=device != "cpu"):
                nxt = model(ids[:, -model.context_length:])[:, -1].argmax(-1, keepdim=True)
            if k == 0:
                torch.cuda.synchronize() if device != "cpu" else None
                ttft.append(time.perf_counter() - t0 - r.arrival)
            ids = torch.cat((ids, nxt), dim=1)
            out_tokens += 1
        served += 1
        if time.perf_counter() - t0 > limit_s:
            break
    wall = time.perf_counter() - t0
    ttft.sort()
    return {"requests": served, "output_tokens": out_tokens, "wall_s": wall, "decode_tok_per_s": out_tokens / wall,
            "ttft_p50_s": ttft[len(ttft) // 2] if ttft else float("nan"), "truncated_after_s": limit_s}


def serve_http(engine, args):
    """Run the engine loop on its own thread and an HTTP front end (uvicorn) in this one until interrupted."""
    import uvicorn
    from llm_systems_from_scratch_b200.serving.server import EngineServer, build_app
    tokenizer = None
    if args.vocab and args.merges:
        from llm_systems_from_scratch_b200.tokenizer.bpe import Tokenizer
        tokenizer = Tokenizer.from_files(args.vocab, args.merges, special_tokens=["<|endoftext|>"])
    engine.set_sampling(args.temperature, args.top_k)       # one setting per server: the decode graphs are captured with it
    server = EngineServer(engine, max_waiting=args.max_waiting).start()
    try:
        uvicorn.run(build_app(server, tokenizer), host=args.host, port=args.http, log_level="info")
    finally:
        server.stop()
    return 0


def main(argv=None):
    from llm_systems_from_scratch_b200.models.transformer import TransformerLM
    from llm_systems_from_scratch_b200.serving import ServingEngine, poisson_trace
    from llm_systems_from_scratch_b200.utils.config import load_config, validate
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default=os.path.join(ROOT, "configures", "serve_1p3b.yaml"))
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--num-requests", type=int, default=None)
    ap.add_argument("--rate", type=float, default=None, help="arrivals per second per GPU")
    ap.add_argument("--offline", action="store_true", help="ignore arrival times (throughput mode)")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--impl", choices=["native", "reference"], default="native")
    ap.add_argument("--time-limit", type=float, default=120.0, help="seconds after which the reference loop stops")
    ap.add_argument("--http", type=int, default=None, metavar="PORT",
                    help="serve POST /generate, GET /health and GET /stats on this port instead of replaying a trace")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--max-waiting", type=int, default=None,
                    help="with --http: refuse (503) submissions while this many requests are already waiting")
    ap.add_argument("--temperature", type=float, default=0.0, help="with --http: 0 = greedy, else sample on the device")
    ap.add_argument("--top-k", type=int, default=None, help="with --http and a temperature: keep the k best logits")
    ap.add_argument("--vocab", default=None, help="tokenizer vocabulary (with --merges: text prompts over HTTP)")
    ap.add_argument("--merges", default=None)
    args = ap.parse_args(argv)
    cfg = validate(load_config(args.config), require_dataset=False)
    m, s = cfg["model"], cfg["serving"]
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    cuda = torch.cuda.is_available()
    device = f"cuda:{local}" if cuda else "cpu"
    if cuda:
        torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl" if cuda else "gloo")
    torch.manual_seed(0)
    keys = ("vocab_size", "context_length", "d_model", "num_layers", "num_heads", "d_ff", "rope_theta")
    trace = poisson_trace(args.num_requests or s["num_requests"], args.rate or s["arrival_rate"], tuple(s["prompt_len"]),
                          tuple(s["output_len"]), m["vocab_size"], seed=s["seed"] + rank)
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        from llm_core.model import TransformerLM as RefLM
        model = RefLM(**{k: m[k] for k in keys}, use_flash_attn=True).to(device).eval()
        res = naive_loop(model, trace, device, args.time_limit)
    else:
        with torch.device(device):
            model = TransformerLM(**{k: m[k] for k in keys}, use_flash_attn=True, use_custom_triton=True)
        if args.checkpoint:
            state = torch.load(args.checkpoint, map_location="cpu")
            model.load_state_dict(state.get("model", state))
        model.eval()
        eng = ServingEngine(model, page_size=s["page_size"], max_batch=s["max_batch"], max_context=s["max_context"],
                            use_cuda_graphs=not args.no_graphs)
        if args.http is not None:
            return serve_http(eng, args)
        eng.warmup()
        res = eng.run(trace, realtime=not args.offline)
    if world > 1:
        import torch.distributed as dist
        gathered = [None] * world
        dist.all_gather_object(gathered, res)
        if rank == 0:
            res = {"requests": sum(g["requests"] for g in gathered), "output_tokens": sum(g["output_tokens"] for g in gathered),
                   "wall_s": max(g["wall_s"] for g in gathered),
                   "decode_tok_per_s": sum(g["output_tokens"] for g in gathered) / max(g["wall_s"] for g in gathered),
                   "ttft_p50_s": sorted(g["ttft_p50_s"] for g in gathered)[world // 2], "per_replica": gathered}
        dist.destroy_process_group()
    if rank == 0:
        res.update(metric="serving_decode_tok_per_s", impl=args.impl, n_gpus=world, model="TransformerLM-1.3B"
                   if m["d_model"] == 2048 else "custom", rate_per_gpu=args.rate or s["arrival_rate"])
        print(json.dumps(res))


if __name__ == "__main__":
    main()
