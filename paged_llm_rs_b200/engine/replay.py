"""Trace replay: feed given token ids through the model step by step and write
the logits.  Nothing is sampled.

It drives the engine's own model, step function, cache manager and kernels, the
ones generation uses; it has no forward pass, cache or loader of its own.  The
reference has no such program; its tests feed given tokens through
``forward_batch`` in the same way (crates/pagedllm/tests/batching.rs:48-64,
265-297).

Input, one JSON object a line on standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits
at the wanted places as little-endian float32 [wanted, vocab].  After every
step a line ``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

PAGE_SIZE = 16
ROUND_TO = 64


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE)
    args = ap.parse_args(argv)

    from .runner import ModelRunner
    from .step import StepEntry

    os.makedirs(args.out, exist_ok=True)
    if ROUND_TO % args.page_size:
        print(f"trace_run: --page-size {args.page_size} does not divide {ROUND_TO}", file=sys.stderr)
        return 2
    pages = max(1, -(-args.max_tokens // args.page_size))
    # Sharing of equal prefixes is off: a replayed request computes every token it is given.
    runner = ModelRunner(args.model, dtype=args.dtype, page_size=args.page_size, num_pages=pages,
                         max_requests=8, prefix_cache=False)
    cache = runner.cache
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if not cache.has(rid):
                cache.open(rid)
            if not cache.reserve(rid, len(e["tokens"])):
                raise SystemExit(f"trace_run: step {rec['step']}: no pages left for request {rid!r} "
                                 f"(--max-tokens {args.max_tokens})")
            entries.append(StepEntry(rid, e["tokens"], e.get("want", [])))
        logits = runner.step(entries)
        for e in entries:
            cache.commit(e.request_id, len(e.tokens))
        if logits.shape[0]:
            logits.cpu().numpy().astype("<f4").tofile(os.path.join(args.out, f"{rec['step']}.f32"))
        for rid in rec.get("end", []):
            if cache.has(rid):
                cache.close(rid)
        print(f"done {rec['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
