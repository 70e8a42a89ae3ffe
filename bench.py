#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of the Qwen3-0.6B shape with random weights
(N(0, 0.02), norm gains 1 + N(0, 0.1)), a batch of 8 and a context of 4096
tokens, in bfloat16.  A "step" is one decode step: every live request gets its
next token.  One JSON line is printed:

  value        decoded tokens a second, K replays of the captured decode step
               timed on the device with CUDA events
  e2e          the same through the Python entry point (Engine.submit / Engine.step):
               host token ids in, host token ids out, every step with its copy of
               the packed step from pinned memory and its copy of the tokens back
  prefill      one prompt of 2048 tokens through the step function
  roofline     bytes the decode step has to read (every weight once and the live
               requests' cache) over its time, against the measured copy bandwidth
  points       decode tokens a second at batch 1 and 64, same context

The engine runs on one GPU: for --gpus above 1 a line says so and the exit code is 2.
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPE_0_6B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu", attention_bias=False,
    hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
    head_dim=128, rms_norm_eps=1e-6, vocab_size=151936, max_position_embeddings=40960, tie_word_embeddings=True,
    rope_theta=1000000.0, sliding_window=None, use_sliding_window=False,
)
# the other two shapes the baseline names, for --shape: the default run and its JSON contract stay the 0.6B one
SHAPE_8B = dict(SHAPE_0_6B, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
                num_key_value_heads=8, tie_word_embeddings=False)
SHAPE_32B = dict(SHAPE_0_6B, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64,
                 num_key_value_heads=8, tie_word_embeddings=False)
SHAPES = {"0.6b": ("Qwen3-0.6B", SHAPE_0_6B), "8b": ("Qwen3-8B", SHAPE_8B), "32b": ("Qwen3-32B", SHAPE_32B)}
PAGE = 16
PREFILL_TOKENS = 2048


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 200 ms while the timed regions run."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.marks = [], None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def region(self, t0, t1):
        self.marks.append((t0, t1))

    def stop(self):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
        inside = [r for t, r in self.rows if any(a - 0.1 <= t <= b + 0.1 for a, b in self.marks)] or [r for _, r in self.rows]
        if not inside:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi gave no samples"])
        sm = [float(r[0]) for r in inside if r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in inside if r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 4 + i and r[4 + i].lower().startswith("active") for r in inside)]
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=reasons, samples=len(inside))


def time_on_device(fn, steps, warmup):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps, (t0, time.time())


def decode_point(runner, batch, context, steps, warmup, clocks):
    """Device time of the captured decode step at ``batch`` requests of ``context`` tokens."""
    import numpy as np
    from paged_llm_rs_b200.engine.step import StepEntry

    cache = runner.cache
    ids = [f"bench{b}" for b in range(batch)]
    for r in ids:
        cache.open(r)
        assert cache.reserve(r, context), "the cache pool is too small for this point"
        cache.commit(r, context - 1)   # the cache holds context-1 tokens (random contents); the step adds one
    entries = [StepEntry(r, [1 + i], [0]) for i, r in enumerate(ids)]
    temp = np.zeros(batch, dtype=np.float32)
    uni = np.zeros(batch, dtype=np.float32)
    runner.step_and_sample(entries, temp, uni)          # packs the step, captures the graph on first use
    graph = runner._decode_graph(entries)
    ms, span = time_on_device(graph.graph.replay, steps, warmup)
    clocks.region(*span)
    launches = graph.launches
    for r in ids:
        cache.close(r)
    return ms, launches


TRACE_KERNELS = {0: "(tcgen05 kernel)", 1: "embed", 2: "rmsnorm", 3: "swiglu", 4: "qk_norm_rope_kv", 5: "attention_generic", 6: "attention_reduce",
                 7: "attention_mma", 8: "attention_tma", 9: "skinny_gemm", 10: "sample_partial", 11: "sample_final", 12: "gemm_tcgen05", 13: "attention_tcgen05"}
TRACE_FILES = ["elementwise", "qk_norm_rope_kv", "attention_generic", "attention_mma", "attention_decode_tma", "sampling",
               "skinny_gemm", "gemm_tcgen05", "attention_prefill_tcgen05"]


def timeline(runner, batch, context, layers, prefill_tokens=0, vocab=1000, mixed_tokens=0) -> int:
    """One replay of the captured decode step, clocked by the kernels themselves (thread 0 of
    each kernel's first CTA reads the global timer before and after its wait for the kernel
    before it).  "to next" is the time from a kernel's wait ending to the next kernel's wait
    ending: what the kernel costs in the chain.  "in place" is how long its first CTA sat on an
    SM before its wait ended.  Library kernels (the output head) carry no stamps: their time
    shows in the "to next" of the kernel before them."""
    import ctypes
    import numpy as np
    import torch
    from paged_llm_rs_b200.engine.step import StepEntry
    from paged_llm_rs_b200.kernels import ops

    lib = ops.lib()
    buf = (ctypes.c_ulonglong * (8192 * 3))()

    def read():
        recs = []
        for f in TRACE_FILES:
            fn = getattr(lib, f"pllm_trace_read_{f}")
            fn.restype = ctypes.c_int
            n = fn(buf, 8192)
            recs += [(buf[3 * i + 2], buf[3 * i + 1], int(buf[3 * i])) for i in range(n)]
        return sorted(recs)

    cache = runner.cache
    if mixed_tokens:
        # a mixed step: the decoding requests beside one portion of a prompt that has 1024 tokens behind it
        ids = [f"t{b}" for b in range(batch)]
        for r in ids:
            cache.open(r)
            assert cache.reserve(r, context)
            cache.commit(r, context - 1)
        cache.open("tp")
        assert cache.reserve("tp", 1024 + mixed_tokens)
        cache.commit("tp", 1024)
        prompt = np.random.default_rng(0).integers(0, vocab, mixed_tokens).tolist()
        entries = [StepEntry(r, [1 + i], [0]) for i, r in enumerate(ids)] + [StepEntry("tp", prompt, [])]
        zeros = np.zeros(batch, dtype=np.float32)
        runner.graph_step_tokens = batch + mixed_tokens
        runner.step_and_sample(entries, zeros, zeros)
        graph = runner._portion_graph(entries)
        assert graph is not None, "the mixed step does not run as a captured step"
    elif prefill_tokens:
        prompt = np.random.default_rng(0).integers(0, vocab, prefill_tokens).tolist()
        cache.open("tp")
        assert cache.reserve("tp", prefill_tokens)
        entries = [StepEntry("tp", prompt, [prefill_tokens - 1])]
        zeros = np.zeros(1, dtype=np.float32)
        runner.step_and_sample(entries, zeros, zeros)
        graph = runner._portion_graph(entries)
        assert graph is not None, "the portion does not run as a captured step"
    else:
        ids = [f"t{b}" for b in range(batch)]
        for r in ids:
            cache.open(r)
            assert cache.reserve(r, context)
            cache.commit(r, context - 1)
        entries = [StepEntry(r, [1 + i], [0]) for i, r in enumerate(ids)]
        zeros = np.zeros(batch, dtype=np.float32)
        runner.step_and_sample(entries, zeros, zeros)
        graph = runner._decode_graph(entries)
    for _ in range(5):
        graph.graph.replay()
    torch.cuda.synchronize()
    read()
    graph.graph.replay()
    torch.cuda.synchronize()
    recs = read()
    rows = []
    for i, (after, before, kid) in enumerate(recs):
        nxt = recs[i + 1][0] if i + 1 < len(recs) else after
        rows.append((TRACE_KERNELS.get(kid, str(kid)), (after - recs[0][0]) / 1e3, (nxt - after) / 1e3, (after - before) / 1e3))
    per_layer = max(1, (len(rows) - 4) // max(1, layers))
    start = min(len(rows), 2 + per_layer * (layers // 2))
    what = f"prefill step, {prefill_tokens} tokens" if prefill_tokens else f"decode step, batch {batch}, context {context}"
    if mixed_tokens:
        what = f"mixed step, {batch} decoding at context {context} beside a portion of {mixed_tokens} tokens"
    print(f"{what}, {layers} layers: {len(rows)} kernels stamped, "
          f"{(recs[-1][0] - recs[0][0]) / 1e3:.1f} us from first to last")
    print(f"one layer from the middle:\n{'kernel':18s} {'at us':>9s} {'to next':>8s} {'in place':>8s}")
    for name, t, d, w in rows[start:start + per_layer]:
        print(f"{name:18s} {t:9.2f} {d:8.2f} {w:8.2f}")
    tot = {}
    for name, t, d, w in rows:
        a = tot.setdefault(name, [0, 0.0, 0.0])
        a[0] += 1; a[1] += d; a[2] += w
    print(f"whole step by kernel:\n{'kernel':18s} {'count':>5s} {'sum us':>9s} {'mean':>7s} {'in place':>8s}")
    for k, (n, d, w) in sorted(tot.items(), key=lambda kv: -kv[1][1]):
        print(f"{k:18s} {n:5d} {d:9.1f} {d / n:7.2f} {w / n:8.2f}")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--shape", choices=sorted(SHAPES), default="0.6b", help="layer sizes: the baseline's 0.6B (default), 8B or 32B shape")
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the shape has (named in config)")
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--timeline-prefill", action="store_true",
                    help="with --only timeline: the captured step of a 2048-token prompt portion instead of the decode step")
    ap.add_argument("--timeline-mixed", type=int, default=0, metavar="TOKENS",
                    help="with --only timeline: the decoding requests beside one prompt portion of this many tokens")
    ap.add_argument("--only", choices=["decode", "prefill", "timeline"], default=None,
                    help="run one part alone and print a short line (for profiling; not a bench record); "
                         "timeline: one captured decode step as the kernels themselves clocked it")
    args = ap.parse_args(argv)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "nicoNaeg/paged-llm-rs is a Rust workspace (cargo, candle): pip cannot install it "
                          "('neither setup.py nor pyproject.toml found') and this image has no cargo or rustc"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    steps, warmup = args.steps, max(3, args.warmup)
    if args.only == "timeline":
        # a build of the kernels that stamps the global timer around each kernel's wait for its predecessor
        os.environ["PAGED_LLM_NVCC_DEFINES"] = (os.environ.get("PAGED_LLM_NVCC_DEFINES", "") + " PLLM_TRACE=1").strip()

    import numpy as np
    import torch
    from paged_llm_rs_b200 import Engine, write_random_model

    pk = peaks()
    shape_name, shape = SHAPES[args.shape][0], dict(SHAPES[args.shape][1])
    layers_full = shape["num_hidden_layers"]
    if args.layers:
        shape["num_hidden_layers"] = args.layers
    B, ctx = args.batch, args.context
    tmp = tempfile.mkdtemp(prefix="pllm_bench_")
    clocks = ClockSampler()
    try:
        model_dir = write_random_model(os.path.join(tmp, "model"), shape, 0, device="cuda")
        most = 1 if (args.no_points or args.only) else 64
        pages = max(most, B) * (ctx // PAGE + 4) + PREFILL_TOKENS // PAGE + 64
        eng = Engine(model_dir, dtype="bfloat16", block_size=PAGE, blocks=pages, max_batch=max(most, B),
                     chunk=PREFILL_TOKENS, prefix_cache=False)
        runner = eng.runner
        for g in runner.cache.groups:       # cache contents for the device-timed points: random, not zeros
            g.pool.normal_(0.0, 1.0)
        L, H, I = shape["num_hidden_layers"], shape["hidden_size"], shape["intermediate_size"]
        nh, nkv, hd, V = shape["num_attention_heads"], shape["num_key_value_heads"], shape["head_dim"], shape["vocab_size"]
        layer_params = H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * I
        weight_bytes = 2 * (L * layer_params + V * H)          # the tied table is read once, as the head
        kv_token_bytes = runner.cache.bytes_per_token()
        clocks.start()

        if args.only == "prefill":
            from paged_llm_rs_b200.engine.step import StepEntry
            prompt = np.random.default_rng(0).integers(0, V, PREFILL_TOKENS).tolist()
            one_zero = np.zeros(1, dtype=np.float32)
            for _ in range(warmup + steps):
                runner.cache.open("prefill")
                runner.cache.reserve("prefill", PREFILL_TOKENS)
                runner.step_and_sample([StepEntry("prefill", prompt, [PREFILL_TOKENS - 1])], one_zero, one_zero)
                runner.cache.close("prefill")
            torch.cuda.synchronize()
            print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "steps": steps}))
            return 0

        if args.only == "timeline":
            return timeline(runner, B, ctx, L, PREFILL_TOKENS if args.timeline_prefill else 0, V, args.timeline_mixed)

        # -- decode, on the device -------------------------------------------------------
        ms, launches = decode_point(runner, B, ctx, steps, warmup, clocks)
        if args.only == "decode":
            print(json.dumps({"only": "decode", "batch": B, "context": ctx, "ms_per_step": round(ms, 4),
                              "launches_per_step": launches}))
            return 0
        value = B / (ms / 1e3)
        step_bytes = weight_bytes + B * ctx * kv_token_bytes
        achieved = step_bytes / (ms / 1e3) / 1e9
        points = {}
        if not args.no_points:
            for b in (1, 64):
                pms, _ = decode_point(runner, b, ctx, max(10, steps // 2), warmup, clocks)
                points[f"decode_b{b}"] = round(b / (pms / 1e3), 1)

        # -- prefill of 2048 tokens ---------------------------------------------------------
        from paged_llm_rs_b200.engine.step import StepEntry
        prompt = np.random.default_rng(0).integers(0, V, PREFILL_TOKENS).tolist()

        one_zero = np.zeros(1, dtype=np.float32)

        def prefill():
            runner.cache.open("prefill")
            runner.cache.reserve("prefill", PREFILL_TOKENS)
            # as the engine runs a prompt's portion: the step and its greedy sample, captured and replayed
            runner.step_and_sample([StepEntry("prefill", prompt, [PREFILL_TOKENS - 1])], one_zero, one_zero)
            runner.cache.close("prefill")

        pms, span = time_on_device(prefill, 5, 3)
        clocks.region(*span)
        flops = 2 * PREFILL_TOKENS * L * layer_params + 2 * PREFILL_TOKENS ** 2 * nh * hd * L + 2 * V * H
        prefill_out = dict(value=round(PREFILL_TOKENS / (pms / 1e3), 1), tokens=PREFILL_TOKENS, ms=round(pms, 3),
                           frac=round(flops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4))

        # -- end to end through the entry point ---------------------------------------------
        rng = np.random.default_rng(1)
        budget = warmup + steps + 2
        for _ in range(B):
            eng.submit(rng.integers(0, V, ctx - budget - 16).tolist(), max_tokens=100000)
        while eng.scheduler.waiting or any(s.prompt_left for s in eng.scheduler.running):
            eng.step()                               # the prompts, untimed
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        h2d = d2h = 0
        t0 = time.time()
        for _ in range(steps):
            out = eng.step()
            h2d += runner.bytes_h2d
            d2h += eng.bytes_d2h
            assert out is not None and len(out.tokens) == B
        torch.cuda.synchronize()
        t1 = time.time()
        clocks.region(t0, t1)
        e2e = dict(value=round(B * steps / (t1 - t0), 1), unit="tokens/s", h2d_bytes_per_step=h2d // steps,
                   d2h_bytes_per_step=d2h // steps, ms_per_step=round((t1 - t0) / steps * 1e3, 4))
        clk = clocks.stop()
    finally:
        shutil.rmtree(tmp, ignore_errors=True)

    line = {
        "metric": f"decode tokens/s ({shape_name} shape, batch {B}, context {ctx})", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {
            "model": f"{shape_name} shape, random weights N(0,0.02) seed 0", "layers": L, "layers_of_shape": layers_full,
            "hidden": H, "heads": nh, "kv_heads": nkv, "head_dim": hd, "intermediate": I, "vocab": V,
            "tie_word_embeddings": bool(shape["tie_word_embeddings"]), "global_batch": B, "seq_len": ctx, "page_size": PAGE,
            "prefill_tokens": PREFILL_TOKENS, "parallelism": "one GPU",
            "l2": f"inputs larger than L2: a step reads {step_bytes / 1e6:.0f} MB",
            "peaks": pk["source"], "hbm_gbs_peak": pk["hbm_gbs"], "bf16_tflops_peak": pk["bf16_tflops"],
        },
        "e2e": e2e, "gpu_launches": launches * steps, "clocks": clk, "prefill": prefill_out,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
