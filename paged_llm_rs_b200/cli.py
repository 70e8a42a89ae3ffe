"""Command line.  Options carry the names, meanings and defaults of the
reference's only binary, its server (crates/pagedllm-server/src/main.rs:20-71):
--model, --dtype {auto,f32,bf16}, --max-tokens 512, --block-size 16,
--cache-mib 3584, --max-batch 16, --attention kernel, --prefix-cache on|off,
--chunk N|off, --require-gpu.  There is no server here: ``generate`` takes token
ids and prints token ids; ``random-model`` writes a model folder from a
config.json and a seed.
"""

from __future__ import annotations

import argparse
import json
import sys


def _chunk(v: str):
    if v == "off":
        return None
    try:
        n = int(v)
    except ValueError:
        raise argparse.ArgumentTypeError(f'--chunk {v!r}, which is neither a token count nor "off"')
    if n == 0:
        raise argparse.ArgumentTypeError("--chunk 0 would carry nothing")
    return n


def _on_off(v: str) -> bool:
    if v not in ("on", "off"):
        raise argparse.ArgumentTypeError(f"{v!r}, which is neither on nor off")
    return v == "on"


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="paged_llm_rs_b200", description="Paged-KV inference engine for one B200")
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate token ids from token ids")
    g.add_argument("--model", required=True, help="directory holding config.json and model.safetensors")
    g.add_argument("--dtype", choices=["auto", "f32", "bf16"], default="auto",
                   help="auto keeps the checkpoint's own dtype")
    g.add_argument("--require-gpu", action="store_true", help="always the case here: there is no CPU path")
    g.add_argument("--max-tokens", type=int, default=512, help="token budget of a request")
    g.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    g.add_argument("--cache-mib", type=int, default=3584, help="bytes the KV cache may take, in MiB")
    g.add_argument("--blocks", type=int, default=None, help="pages in the pool, instead of --cache-mib")
    g.add_argument("--max-batch", type=int, default=16, help="rows in one decode step")
    g.add_argument("--attention", default="kernel", choices=["kernel", "tensor"])
    g.add_argument("--prefix-cache", type=_on_off, default=True, metavar="on|off")
    g.add_argument("--chunk", type=_chunk, default=128, metavar="N|off",
                   help="most tokens one step may carry; off runs a prompt whole")
    g.add_argument("--max-prefill-seqs", type=int, default=1,
                   help="prompts that may share one pass in chunked mode (1: one joins per pass, as in the reference)")
    g.add_argument("--prompt-ids", action="append", default=[], metavar="1,2,3",
                   help="one prompt as comma-separated token ids; may be given several times")
    g.add_argument("--prompts-file", help="JSON file with a list of prompts, each a list of token ids")
    g.add_argument("--prompt-len", type=int, action="append", default=[], metavar="N",
                   help="one prompt of N uniform-random token ids drawn from --seed; may be given several times")
    g.add_argument("--reference-draw-order", action="store_true",
                   help="draw plain temperature requests on the host in the reference's order (falling probability), "
                        "so that a seed gives the reference's tokens; default: on the device, token ids upward")
    g.add_argument("--temperature", type=float, default=None)
    g.add_argument("--top-k", type=int, default=None)
    g.add_argument("--top-p", type=float, default=None)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--stop-ids", default="", help="comma-separated stop token ids (default: the model's eos ids)")
    g.add_argument("--metrics", action="store_true", help="print the scheduler's counters to stderr")

    r = sub.add_parser("random-model", help="write a model folder with random weights")
    r.add_argument("--config", required=True, help="a config.json to read sizes from")
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--dtype", choices=["f32", "bf16"], default="bf16")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.command == "random-model":
        import torch
        from .config.schema import read_json
        from .weights.random_init import write_random_model

        write_random_model(args.out, read_json(args.config), args.seed,
                           torch.float32 if args.dtype == "f32" else torch.bfloat16)
        print(args.out)
        return 0

    from .config.schema import GenerationDefaults
    from .engine.engine import Engine
    from .weights.safetensors_io import open_model_files

    if args.attention == "tensor":
        print("--attention tensor: this engine has no gathered-tensor path; the kernel reads the pages in place",
              file=sys.stderr)
        return 2
    prompts = [[int(x) for x in p.split(",") if x.strip()] for p in args.prompt_ids]
    if args.prompts_file:
        with open(args.prompts_file) as f:
            prompts += json.load(f)
    if not prompts and not args.prompt_len:
        print("no prompt: give --prompt-ids, --prompts-file or --prompt-len", file=sys.stderr)
        return 2
    dtype = args.dtype
    if dtype == "auto":  # the checkpoint's own dtype, read from the embedding (model/mod.rs:175)
        import torch
        files = open_model_files(args.model)
        stored = next((f.dtype(n) for f in files for n in f.names() if n.endswith("embed_tokens.weight")), torch.bfloat16)
        dtype = "f32" if stored == torch.float32 else "bf16"
    defaults = GenerationDefaults.from_dir(args.model)
    temperature = args.temperature if args.temperature is not None else (defaults.temperature or 0.0)
    top_k = args.top_k if args.top_k is not None else defaults.top_k
    top_p = args.top_p if args.top_p is not None else defaults.top_p
    stop = [int(x) for x in args.stop_ids.split(",") if x.strip()] or list(defaults.eos_token_ids)
    engine = Engine(args.model, dtype=dtype, block_size=args.block_size, cache_mib=args.cache_mib, blocks=args.blocks,
                    max_batch=args.max_batch, chunk=args.chunk, prefix_cache=args.prefix_cache,
                    max_prefill_seqs=args.max_prefill_seqs, reference_draw_order=args.reference_draw_order)
    if args.prompt_len:
        import numpy as np
        rng = np.random.default_rng(args.seed)
        prompts += [rng.integers(0, engine.runner.vocab_size, n).tolist() for n in args.prompt_len]
    cache = engine.runner.cache
    print(f"model {args.model}  dtype {dtype}  cache {cache.num_pages} pages of {cache.page_size} tokens, "
          f"{cache.bytes_per_token()} bytes a token  chunk {args.chunk or 'off'}  "
          f"prefix cache {'on' if cache.prefix_cache else 'off'}", file=sys.stderr)
    outs = engine.generate(prompts, max_tokens=args.max_tokens, temperature=temperature, top_k=top_k, top_p=top_p,
                           seed=args.seed, stop_tokens=stop)
    for o in outs:
        print(",".join(str(t) for t in o))
    if args.metrics:
        print(json.dumps(engine.metrics()), file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
