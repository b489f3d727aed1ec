"""Command line in the reference's manner: single-dash Go-style flags.

Flags that the reference has keep its names and meanings (cmd/neurogrid/main.go:884-898):
``-model`` path to the model folder, ``-gpu`` device id, ``-max-seq-len`` cap on the context
and the cache.  Its server, peer-to-peer and speculative flags have no meaning for one
engine on one GPU.  Added here: a random-weights mode, the compute dtype, cache and
scheduler sizes, and a prompt given as token ids (the engine works on token ids; there is no
tokenizer).
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List, Optional


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="neurogrid", description="LFM2 inference on one B200 (token ids in, token ids out)")
    a = ap.add_argument
    a("-model", "--model", default="", help="Path to model weights (folder with config.json and safetensors)")
    a("-gpu", "--gpu", type=int, default=0, help="Local GPU device ID")
    a("-max-seq-len", "--max-seq-len", type=int, default=4096,
      help="Maximum sequence length for KV cache (caps model's max_position_embeddings to save VRAM)")
    a("-random-weights", "--random-weights", type=int, default=None, metavar="SEED",
      help="Draw random weights from SEED (with -config); with -write-model, write them as a model folder")
    a("-config", "--config", default="", help="config.json to use with -random-weights")
    a("-write-model", "--write-model", default="", metavar="DIR",
      help="Write config.json and model.safetensors for -config and -random-weights into DIR, then exit")
    a("-dtype", "--dtype", default="bf16", choices=["bf16", "bfloat16", "fp32", "float32"], help="Compute dtype")
    a("-page-size", "--page-size", type=int, default=16, help="Tokens per cache page")
    a("-num-pages", "--num-pages", type=int, default=None, help="Pages in the cache pool (default: from memory)")
    a("-max-requests", "--max-requests", type=int, default=8, help="Requests live at a time")
    a("-max-tokens-per-step", "--max-tokens-per-step", type=int, default=2048, help="Token budget of a step")
    a("-chunk-size", "--chunk-size", type=int, default=None, help="Longest prompt portion in a step")
    a("-prompt-tokens", "--prompt-tokens", action="append", default=[], metavar="IDS",
      help='Prompt as comma-separated token ids, e.g. "1,2,3" (repeatable: one request each)')
    a("-prompt-len", "--prompt-len", type=int, action="append", default=[], metavar="N",
      help="A prompt of N random token ids drawn from -seed (repeatable)")
    a("-max-new-tokens", "--max-new-tokens", type=int, default=16, help="Tokens to generate per request")
    a("-temperature", "--temperature", type=float, default=0.0, help="Sampling temperature (<= 0: greedy)")
    a("-top-p", "--top-p", type=float, default=1.0, help="Nucleus sampling mass")
    a("-seed", "--seed", type=int, default=42, help="Seed of the sampler (and of random prompts)")
    a("-ignore-eos", "--ignore-eos", action="store_true", help="Do not stop at the model's EOS token")
    a("-log-level", "--log-level", default="info", choices=["debug", "info", "warn", "error"], help="Log level")
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    log = (lambda *a: print(*a, file=sys.stderr, flush=True)) if args.log_level in ("debug", "info") else (lambda *a: None)
    config = None
    if args.config:
        with open(args.config) as f:
            config = json.load(f)
    if args.write_model:
        if config is None or args.random_weights is None:
            print("-write-model needs -config and -random-weights", file=sys.stderr)
            return 2
        from .weights import write_random_model
        write_random_model(config, args.random_weights, args.write_model)
        log(f"wrote {args.write_model}")
        return 0
    if not args.model and (config is None or args.random_weights is None):
        print("give -model DIR, or -config FILE with -random-weights SEED", file=sys.stderr)
        return 2
    import torch
    from .engine.api import Engine
    t0 = time.time()
    eng = Engine(args.model or None, config=config, random_weights=args.random_weights, dtype=args.dtype,
                 gpu=args.gpu, max_seq_len=args.max_seq_len, page_size=args.page_size, num_pages=args.num_pages,
                 max_requests=args.max_requests, max_tokens_per_step=args.max_tokens_per_step,
                 chunk_size=args.chunk_size)
    log(f"model ready in {time.time() - t0:.1f} s: {eng.model.spec.architecture}, "
        f"{eng.model.weight_bytes() / 1e6:.1f} MB of weights, {eng.runner.cache.pools[0].num_pages if eng.runner.cache.pools else 0} pages")
    prompts = [[int(x) for x in p.replace(" ", "").split(",") if x] for p in args.prompt_tokens]
    gen = torch.Generator().manual_seed(args.seed)
    for n in args.prompt_len:
        prompts.append(torch.randint(0, eng.model.spec.vocab_size, (n,), generator=gen).tolist())
    if not prompts:
        print("no prompt: give -prompt-tokens or -prompt-len", file=sys.stderr)
        return 2
    t0 = time.time()
    outs = eng.generate(prompts, max_new_tokens=args.max_new_tokens, temperature=args.temperature,
                        top_p=args.top_p, seed=args.seed, ignore_eos=args.ignore_eos)
    dt = time.time() - t0
    for i, (o, why) in enumerate(zip(outs, eng.last_finish_reasons)):
        print(json.dumps({"request": i, "tokens": o, "finish_reason": why}))
    n = sum(len(o) for o in outs)
    log(f"{n} tokens in {dt:.3f} s ({n / dt:.1f} tok/s incl. prefill); {eng.stats()}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
