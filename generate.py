#!/usr/bin/env python
"""Interactive text generation from a trained checkpoint.

Same flags as the reference REPL (generate.py:7-60).  ``--temperature 0`` decodes greedily and
``--top-k`` really filters.  A prompt can also be given with ``--prompt`` for non-interactive use.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from llm_systems_from_scratch_b200.models.transformer import TransformerLM  # noqa: E402
from llm_systems_from_scratch_b200.tokenizer.bpe import Tokenizer  # noqa: E402


def complete(model, tokenizer, prompt: str, device, max_tokens: int, temperature: float, top_k, eos_id):
    ids = torch.tensor([tokenizer.encode(prompt)], dtype=torch.long, device=device)
    out = model.generate(ids, max_new_tokens=max_tokens, temperature=temperature, top_k=top_k, eos_token_id=eos_id)
    return tokenizer.decode(out.reshape(-1).tolist())


def main(argv=None):
    ap = argparse.ArgumentParser(description="Generate text from a pretrained model")
    ap.add_argument("--config", type=str, default="model_config.json")
    ap.add_argument("--checkpoint", type=str, default="ckpt_final.pt")
    ap.add_argument("--vocab", type=str, default="vocab.json")
    ap.add_argument("--merges", type=str, default="merges.json")
    ap.add_argument("--max-tokens", type=int, default=200)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=None)
    ap.add_argument("--device", type=str, default="auto")
    ap.add_argument("--prompt", type=str, default=None, help="generate once for this prompt and exit")
    args = ap.parse_args(argv)
    device = ("cuda" if torch.cuda.is_available() else "cpu") if args.device == "auto" else args.device
    model = TransformerLM.from_pretrained(config_path=args.config, checkpoint_path=args.checkpoint).to(device)
    model.eval()
    tokenizer = Tokenizer.from_files(args.vocab, args.merges, special_tokens=["<|endoftext|>"])
    eos_id = tokenizer.encode("<|endoftext|>")[0]
    if args.prompt is not None:
        print(complete(model, tokenizer, args.prompt, device, args.max_tokens, args.temperature, args.top_k, eos_id))
        return
    print("Model loaded. Type your prompt (Ctrl+C to quit):\n")
    while True:
        try:
            prompt = input("> ")
        except (KeyboardInterrupt, EOFError):
            print()
            break
        if prompt:
            print(complete(model, tokenizer, prompt, device, args.max_tokens, args.temperature, args.top_k, eos_id))
            print()


if __name__ == "__main__":
    main()
