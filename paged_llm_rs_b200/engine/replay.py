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

Beyond that contract, for the tests: ``--page-size`` (a divisor of 64),
``--prefix-cache on`` (a request's first entry claims the pages that already hold
its leading tokens, as the scheduler's admission does, crates/pagedllm/src/scheduler.rs:596-621,
and pages are named when a step is committed) and ``--graphs on`` (steps run as
captured and replayed CUDA graphs with the sampling kernel behind them, the way
generation runs them; the chosen tokens are dropped).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

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
    ap.add_argument("--prefix-cache", choices=["on", "off"], default="off",
                    help="on: a request's first entry takes the pages that already hold its leading tokens "
                         "(never a page with a wanted place in it, never its last page) and runs the rest; "
                         "<out>/prefix.json then says how many tokens each request found")
    ap.add_argument("--graphs", choices=["on", "off"], default="off",
                    help="on: steps run as generation runs them: steps of single tokens (each wanted) as the "
                         "replayed captured step, steps that fill more than half of --step-tokens as the "
                         "captured portion step, with the greedy sampling kernel behind them")
    ap.add_argument("--step-tokens", type=int, default=None, help="with --graphs on: the token budget of a captured portion step")
    args = ap.parse_args(argv)

    import numpy as np

    from .runner import ModelRunner
    from .step import StepEntry

    os.makedirs(args.out, exist_ok=True)
    if ROUND_TO % args.page_size:
        print(f"trace_run: --page-size {args.page_size} does not divide {ROUND_TO}", file=sys.stderr)
        return 2
    pages = max(1, -(-args.max_tokens // args.page_size))
    sharing = args.prefix_cache == "on"
    graphs = args.graphs == "on"
    # Unless asked for, sharing of equal prefixes is off: a replayed request computes every token it is given.
    runner = ModelRunner(args.model, dtype=args.dtype, page_size=args.page_size, num_pages=pages,
                         max_requests=8, prefix_cache=sharing, use_graphs=graphs)
    if graphs and args.step_tokens:
        runner.graph_step_tokens = args.step_tokens
    cache = runner.cache
    if sharing and not cache.prefix_cache:
        print("trace_run: this model's caches cannot share prefixes (a window, or state of fixed size)", file=sys.stderr)
        return 2
    history = {}      # request -> every token it has been given
    found = {}        # request -> tokens its first entry found in the cache
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        entries, written = [], []
        for e in rec.get("entries", []):
            rid, tokens, want = e["id"], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]
            skip = 0
            if not cache.has(rid):
                cache.open(rid)
                history[rid] = []
                if sharing:
                    # pages that hold a wanted place are computed, so that its logits exist
                    upto = min(want) + 1 if want else len(tokens)
                    skip = cache.claim_prefix(rid, tokens[:upto])
                    found[rid] = skip
            history[rid] += tokens
            if not cache.reserve(rid, len(tokens) - skip):
                raise SystemExit(f"trace_run: step {rec['step']}: no pages left for request {rid!r} "
                                 f"(--max-tokens {args.max_tokens})")
            entries.append(StepEntry(rid, tokens[skip:], [w - skip for w in want]))
            written.append(len(tokens) - skip)
        if graphs:
            n = sum(len(e.want) for e in entries)
            zeros = np.zeros(max(n, 1), dtype=np.float32)
            logits, _ = runner.step_and_sample(entries, zeros[:n], zeros[:n])
            logits = logits.cpu()
            runner.check_status()
        else:
            logits = runner.step(entries).cpu()
        for e, n in zip(entries, written):
            cache.commit(e.request_id, n, history[e.request_id] if sharing else None)
        if logits.shape[0]:
            logits.numpy().astype("<f4").tofile(os.path.join(args.out, f"{rec['step']}.f32"))
        for rid in rec.get("end", []):
            if cache.has(rid):
                cache.close(rid)
                history.pop(rid, None)
        if sharing:
            a = cache.groups[0].allocator
            with open(os.path.join(args.out, "prefix.json"), "w") as f:
                json.dump(dict(cached_tokens=found, hits=a.hits, misses=a.misses, evictions=a.evictions), f)
        print(f"done {rec['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
