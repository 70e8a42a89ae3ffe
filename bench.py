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
               the packed step from pinned memory and its copy of the tokens back; five
               timed rounds of K steps, the last of which (the K positions before the
               context) is the one reported and the others its spread
  prefill      one prompt of 2048 tokens through the step function (frac: of the library product's burst rate;
               frac_sustained: of its rate in a seconds-long loop under the power cap)
  roofline     bytes the decode step has to read (every weight once and the live
               requests' cache) over its time, against the measured copy bandwidth
  points       decode tokens a second at batch 1 and 64 at the same context, and at batch 1, 8 and 64
               at context 512 (right after the baseline's 512-token prompts), each with its fraction
               of the HBM roofline
  generate     whole generations through Engine.generate by the wall clock: 64 prompts of 512 tokens,
               128 new tokens each, steps of at most 2048 tokens (the first call, which captures its
               steps, is not counted)
  repeats      the spread of the timed region: it is repeated ten times (median, min, max)
  shapes       the same figures at the baseline's 8B shape (36 of 36 layers; with its mixed step: 64
               requests decoding at context 4096 beside a 512-token portion) and at the 32B shape's
               layer sizes (16 of 64 layers, named)
  reference_kernel   the reference's own CUDA kernel (paged_attention.cu, compiled unchanged for
               sm_100a) against this engine's decode attention on the same keys and values

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
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


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


REF_KERNEL = os.path.join(ROOT, "baseline", "_ref", "crates", "pagedllm", "src", "kernels", "paged_attention.cu")


def reference_kernel_points(clocks, reps=10):
    """The reference's one CUDA kernel (crates/pagedllm/src/kernels/paged_attention.cu, compiled unchanged for
    sm_100a with -DELEM=__nv_bfloat16 and launched as crates/pagedllm/src/kernels/paged_attention.rs:626-634,
    684-688 launches it: grid (heads, rows), 128 threads, (blocks x block size + 128) floats of shared memory)
    against this engine's decode attention (the bulk-copy kernel and the reduction of its splits) on the same
    random keys, values and queries, each in its own cache layout.  Microseconds a launch, median of ``reps``."""
    import ctypes
    import subprocess as sp
    import numpy as np
    import torch
    from paged_llm_rs_b200.kernels import attention_plan, ops
    from paged_llm_rs_b200.parts.base import AttentionWork

    if not os.path.exists(REF_KERNEL):
        return {"unavailable": "baseline/_ref holds no copy of the reference's paged_attention.cu"}
    try:
        from cuda.bindings import driver
    except Exception as e:     # noqa: BLE001
        return {"unavailable": f"cuda-python is not importable: {e}"}
    tmp = tempfile.mkdtemp(prefix="pllm_ref_kernel_")
    try:
        cubin = os.path.join(tmp, "paged_attention.cubin")
        r = sp.run(["nvcc", "-cubin", "-arch=sm_100a", "-DELEM=__nv_bfloat16", REF_KERNEL, "-o", cubin],
                   capture_output=True, text=True)
        if r.returncode != 0:
            return {"unavailable": "nvcc failed on the reference's kernel: " + r.stderr.strip()[-200:]}
        torch.zeros(1, device="cuda")                      # the primary context, current
        err, module = driver.cuModuleLoadData(open(cubin, "rb").read())
        if int(err) != 0:
            return {"unavailable": f"cuModuleLoadData: {err}"}
        err, fn = driver.cuModuleGetFunction(module, b"paged_attention_decode")
        if int(err) != 0:
            return {"unavailable": f"cuModuleGetFunction: {err}"}
    finally:
        shutil.rmtree(tmp, ignore_errors=True)

    dev, page = "cuda", PAGE
    out = {}
    g = torch.Generator(device=dev).manual_seed(0)
    sm2 = 2 * torch.cuda.get_device_properties(0).multi_processor_count

    def timed(fn_):
        for _ in range(3):
            fn_()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            flush_l2()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn_(); b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return statistics.median(ts)

    worst = 0.0
    for nh, nkv, hd, tag in ((16, 8, 128, "h16"), (32, 8, 128, "h32")):
        for ctx in (512, 4096):
            for B in (1, 8, 64):
                n_blocks = ctx // page
                tokens = B * ctx
                k = torch.randn(tokens, nkv, hd, device=dev, generator=g).bfloat16()
                v = torch.randn(tokens, nkv, hd, device=dev, generator=g).bfloat16()
                q = torch.randn(B, nh * hd, device=dev, generator=g).bfloat16()
                # pages in a shuffled order, the same order in both layouts
                perm = torch.randperm(B * n_blocks, device=dev, generator=g).to(torch.int32).view(B, n_blocks)
                # the reference's layout: [slots, kv_heads * head_dim], slot = block * block_size + offset
                slot_of = (perm.long()[:, :, None] * page + torch.arange(page, device=dev)[None, None]).view(-1)
                rk = torch.empty(tokens, nkv * hd, device=dev, dtype=torch.bfloat16)
                rv = torch.empty_like(rk)
                rk[slot_of] = k.view(tokens, -1); rv[slot_of] = v.view(tokens, -1)
                table_u32 = perm.contiguous()
                lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
                r_out = torch.zeros(B, nh * hd, device=dev, dtype=torch.bfloat16)
                shared = (n_blocks * page + 128) * 4
                assert shared <= 48 << 10
                stream = torch.cuda.current_stream().cuda_stream
                vals = (q.data_ptr(), rk.data_ptr(), rv.data_ptr(), table_u32.data_ptr(), lens.data_ptr(), r_out.data_ptr(),
                        page, hd, nh, nkv, n_blocks, 128, 4, float(hd ** -0.5))
                types = (ctypes.c_void_p,) * 6 + (ctypes.c_uint,) * 7 + (ctypes.c_float,)

                def ref():
                    (e,) = driver.cuLaunchKernel(fn, nh, B, 1, 128, 1, 1, shared, stream, (vals, types), 0)
                    assert int(e) == 0, e
                # this engine's layout: [pages, kv_heads, page, head_dim], rows swizzled
                kp = k.view(B * n_blocks, page, nkv, hd).transpose(1, 2).contiguous()
                vp = v.view(B * n_blocks, page, nkv, hd).transpose(1, 2).contiguous()
                ok = torch.empty_like(kp); ov = torch.empty_like(vp)
                ok[perm.view(-1).long()] = kp; ov[perm.view(-1).long()] = vp
                ops.swizzle_pool_(ok); ops.swizzle_pool_(ov)
                work, red, parts = attention_plan.plan_attention([(i, 1, ctx - 1) for i in range(B)], 1, None, nkv, sm2)
                wd = torch.from_numpy(np.ascontiguousarray(work)).to(dev)
                rd = torch.from_numpy(np.ascontiguousarray(red)).to(dev) if len(red) else torch.zeros(1, 4, dtype=torch.int32, device=dev)
                nw = torch.tensor([len(work)], dtype=torch.int32, device=dev)
                nr = torch.tensor([len(red)], dtype=torch.int32, device=dev)
                po = torch.zeros(max(parts, 1), nh, hd, device=dev)
                pm = torch.zeros(max(parts, 1), nh, 2, device=dev)
                o_out = torch.zeros_like(r_out)
                st = torch.zeros(1, dtype=torch.int32, device=dev)

                plan = AttentionWork(wd, nw, len(work), rd, nr, len(red), po, pm, kinds=1,
                                     many_splits=attention_plan.many_splits(B, nkv, sm2))

                def ours():
                    ops.paged_attention(q, ok, ov, perm, plan, o_out, nh, nkv, hd, 0, hd ** -0.5, st, swizzled=True)
                t0 = time.time()
                t_ref, t_ours = timed(ref), timed(ours)
                clocks.region(t0, time.time())
                assert int(st.item()) == 0
                worst = max(worst, float((r_out.float() - o_out.float()).abs().max()))
                key = f"{tag}_b{B}_ctx{ctx}"
                out[key + "_ref_us"] = round(t_ref, 1)
                out[key + "_ours_us"] = round(t_ours, 1)
                del k, v, rk, rv, kp, vp, ok, ov
    out["max_abs_diff"] = round(worst, 5)
    out["what"] = ("decode attention alone, microseconds a launch (ours: attention + reduction of splits), cold L2; "
                   "h16 = 16 query heads over 8 kv heads of 128 (0.6B), h32 = 32 over 8 (8B)")
    return out


_FLUSH = None


def flush_l2():
    """Write a buffer larger than the 126 MB L2."""
    import torch
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.fill_(1)


def time_on_device(fn, steps, warmup, repeats=0):
    """``warmup`` untimed calls, then exactly ``steps`` calls between two events (the contract's timed
    region); then, for the spread, ``repeats`` more such regions.  Returns (ms a call in the first
    region, (wall start, wall end), {"n", "median_ms", "min_ms", "max_ms"} over all regions)."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    per = []
    t0 = time.time()
    for _ in range(1 + repeats):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        per.append(a.elapsed_time(b) / steps)
    spread = dict(n=len(per), median_ms=round(statistics.median(per), 4), min_ms=round(min(per), 4), max_ms=round(max(per), 4))
    return per[0], (t0, time.time()), spread


def decode_point(runner, batch, context, steps, warmup, clocks, repeats=9):
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
    ms, span, spread = time_on_device(graph.replay, steps, warmup, repeats)
    clocks.region(*span)
    launches = graph.launches
    for r in ids:
        cache.close(r)
    return ms, launches, spread


def mixed_point(runner, decoding, context, portion, behind, vocab, steps, warmup, clocks, repeats=9):
    """Device time of one captured mixed step: ``decoding`` requests at ``context`` tokens take their next
    token beside a portion of ``portion`` prompt tokens that has ``behind`` tokens of its prompt before it."""
    import numpy as np
    from paged_llm_rs_b200.engine.step import StepEntry

    cache = runner.cache
    ids = [f"mix{b}" for b in range(decoding)]
    for r in ids:
        cache.open(r)
        assert cache.reserve(r, context)
        cache.commit(r, context - 1)
    cache.open("mixp")
    assert cache.reserve("mixp", behind + portion)
    cache.commit("mixp", behind)
    prompt = np.random.default_rng(0).integers(0, vocab, portion).tolist()
    entries = [StepEntry(r, [1 + i], [0]) for i, r in enumerate(ids)] + [StepEntry("mixp", prompt, [])]
    zeros = np.zeros(decoding, dtype=np.float32)
    was = runner.graph_step_tokens
    runner.graph_step_tokens = decoding + portion
    try:
        runner.step_and_sample(entries, zeros, zeros)
        graph = runner._portion_graph(entries)
        assert graph is not None, "the mixed step does not run as a captured step"
        ms, span, spread = time_on_device(graph.replay, steps, warmup, repeats)
    finally:
        runner.graph_step_tokens = was
    clocks.region(*span)
    for r in ids + ["mixp"]:
        cache.close(r)
    return ms, spread


def prefill_point(runner, vocab, clocks, repeats=9):
    """One prompt of PREFILL_TOKENS tokens through the step function, as the engine runs a prompt's portion:
    the step and its greedy sample, captured and replayed, host packing included."""
    import numpy as np
    from paged_llm_rs_b200.engine.step import StepEntry

    prompt = np.random.default_rng(0).integers(0, vocab, PREFILL_TOKENS).tolist()
    one_zero = np.zeros(1, dtype=np.float32)

    def prefill():
        runner.cache.open("prefill")
        runner.cache.reserve("prefill", PREFILL_TOKENS)
        runner.step_and_sample([StepEntry("prefill", prompt, [PREFILL_TOKENS - 1])], one_zero, one_zero)
        runner.cache.close("prefill")

    # five prompts to a timed region: the host packs the next step while the GPU runs this one
    ms, span, spread = time_on_device(prefill, 5, 3, repeats)
    clocks.region(*span)
    return spread["median_ms"], spread


def generate_point(model_dir, vocab, clocks, requests=64, prompt=512, new=128, repeats=3):
    """Whole generations through ``Engine.generate``: ``requests`` random prompts of ``prompt`` tokens, ``new``
    tokens each, greedy, no stop token; host token lists in and out, by the wall clock.  The first call
    captures the steps it needs and is not counted.  What the scheduler, the portions under the token
    budget, the step packing and the copies cost shows as the gap to the device-timed points."""
    import numpy as np
    import torch
    from paged_llm_rs_b200 import Engine
    eng = Engine(model_dir, dtype="bfloat16", block_size=PAGE, blocks=requests * ((prompt + new) // PAGE + 2) + 64,
                 max_batch=requests, chunk=PREFILL_TOKENS, prefix_cache=False,
                 max_prefill_seqs=max(1, PREFILL_TOKENS // prompt))    # (the token budget decides, not the count)
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, vocab, prompt).tolist() for _ in range(requests)]
    eng.generate(prompts, max_tokens=new, stop_tokens=())
    torch.cuda.synchronize()
    per = []
    for _ in range(repeats):
        t0 = time.time()
        outs = eng.generate(prompts, max_tokens=new, stop_tokens=())
        torch.cuda.synchronize()
        t1 = time.time()
        clocks.region(t0, t1)
        assert all(len(o) == new for o in outs)
        per.append((t1 - t0) * 1e3)
    ms = statistics.median(per)
    m = eng.scheduler.metrics
    return dict(requests=requests, prompt_tokens=prompt, new_tokens=new, ms=round(ms, 1), min_ms=round(min(per), 1),
                max_ms=round(max(per), 1), generated_tokens_s=round(requests * new / (ms / 1e3), 1),
                all_tokens_s=round(requests * (prompt + new) / (ms / 1e3), 1), step_token_budget=PREFILL_TOKENS,
                steps_per_call=m.steps // (repeats + 1))


def long_prompt_points(runner, sizes, total, clocks):
    """A prompt of ``total`` tokens through the step function in portions of 2048: each portion's device time, and
    the fraction of the tensor peak its flops make (the products of 2048 rows, and the attention over everything
    before the portion and half of itself)."""
    import numpy as np
    import torch
    from paged_llm_rs_b200.engine.step import StepEntry
    T, cache, pk = PREFILL_TOKENS, runner.cache, peaks()
    L, nh, hd, V, H = sizes["L"], sizes["nh"], sizes["hd"], sizes["V"], sizes["H"]
    products = sizes["prefill_flops"] - 2 * V * H - 2 * T * T * nh * hd * L        # of a portion's 2048 rows
    prompt = np.random.default_rng(0).integers(0, V, total).tolist()
    zero = np.zeros(1, dtype=np.float32)
    out = {}
    for rep in range(2):                         # (the first pass captures the steps)
        cache.open("long")
        events = []
        t0 = time.time()
        for c in range(0, total, T):
            assert cache.reserve("long", T)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            runner.step_and_sample([StepEntry("long", prompt[c:c + T], [T - 1])], zero, zero)
            b.record()
            events.append((c, a, b))
            cache.commit("long", T)
        torch.cuda.synchronize()
        clocks.region(t0, time.time())
        cache.close("long")
    for c, a, b in events:
        if c % 8192 == 0 or c == total - T:
            ms = a.elapsed_time(b)
            attention = 4 * T * (c + T / 2) * nh * hd * L
            flops = products + attention + 2 * V * H
            out[f"portion_at_{c}"] = dict(ms=round(ms, 3), tokens_s=round(T / ms * 1e3, 1), attention_share_of_flops=round(attention / flops, 3),
                                          bf16_frac=round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4))
    out["whole_prompt_ms"] = round(sum(a.elapsed_time(b) for _, a, b in events), 1)
    out["tokens"] = total
    return out


def shape_sizes(shape):
    L, H, I = shape["num_hidden_layers"], shape["hidden_size"], shape["intermediate_size"]
    nh, nkv, hd, V = shape["num_attention_heads"], shape["num_key_value_heads"], shape["head_dim"], shape["vocab_size"]
    layer_params = H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * I
    return dict(L=L, H=H, I=I, nh=nh, nkv=nkv, hd=hd, V=V, layer_params=layer_params,
                weight_bytes=2 * (L * layer_params + V * H),          # a tied table is read once, as the head
                kv_token_bytes=2 * L * nkv * hd * 2,
                prefill_flops=2 * PREFILL_TOKENS * L * layer_params + 2 * PREFILL_TOKENS ** 2 * nh * hd * L + 2 * V * H)


def scratch_dir():
    """Where the random model folder is written: memory-backed when there is room (a 16 GB file is written
    and read back once), else the temporary folder."""
    try:
        if shutil.disk_usage("/dev/shm").free > (40 << 30):
            return "/dev/shm"
    except OSError:
        pass
    return None


def other_shape(key, layers, pk, clocks, steps, warmup):
    """Decode at batch 1, 8 and 64 (contexts 4096 and 512), the 2048-token prefill and, for the 8B shape, the
    baseline's mixed step, at another of the baseline's shapes: flat figures with their roofline fractions."""
    import gc
    import torch
    from paged_llm_rs_b200 import Engine, write_random_model

    name, shape = SHAPES[key][0], dict(SHAPES[key][1])
    full = shape["num_hidden_layers"]
    shape["num_hidden_layers"] = layers or full
    z = shape_sizes(shape)
    out = {f"{key}_layers": z["L"], f"{key}_layers_of_shape": full}
    tmp = tempfile.mkdtemp(prefix="pllm_bench_", dir=scratch_dir())
    try:
        model_dir = write_random_model(os.path.join(tmp, "model"), shape, 0, device="cuda")
        ctx = 4096
        pages = 64 * (ctx // PAGE + 4) + (PREFILL_TOKENS + 1024) // PAGE + 64
        eng = Engine(model_dir, dtype="bfloat16", block_size=PAGE, blocks=pages, max_batch=64, chunk=PREFILL_TOKENS,
                     prefix_cache=False)
        shutil.rmtree(tmp, ignore_errors=True)
        runner = eng.runner
        for g in runner.cache.groups:
            g.pool.normal_(0.0, 1.0)
        for c in (4096, 512):
            for b in (1, 8, 64):
                ms, _, spread = decode_point(runner, b, c, max(5, steps // 2), warmup, clocks, repeats=4)
                ms = spread["median_ms"]
                gbs = (z["weight_bytes"] + b * c * z["kv_token_bytes"]) / (ms / 1e3) / 1e9
                tag = f"{key}_decode_b{b}" + ("" if c == 4096 else f"_ctx{c}")
                out[tag] = round(b / (ms / 1e3), 1)
                out[tag + "_hbm_frac"] = round(gbs / pk["hbm_gbs"], 4)
        pms, _ = prefill_point(runner, z["V"], clocks, repeats=4)
        out[f"{key}_prefill_tok_s"] = round(PREFILL_TOKENS / (pms / 1e3), 1)
        out[f"{key}_prefill_ms"] = round(pms, 3)
        out[f"{key}_prefill_bf16_frac"] = round(z["prefill_flops"] / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)
        # (against the library product's rate in a seconds-long loop under the power cap: these steps of 26 ms and more,
        #  five to a timed region, run at those clocks)
        out[f"{key}_prefill_bf16_frac_sustained"] = round(z["prefill_flops"] / (pms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
        if key == "8b":
            # the baseline's workload for this shape: 64 requests decoding at context 4096 beside a 512-token
            # portion of a 2048-token prompt (its third portion: 1024 tokens behind it)
            mms, spread = mixed_point(runner, 64, ctx, 512, 1024, z["V"], max(3, steps // 4), warmup, clocks, repeats=4)
            mms = spread["median_ms"]
            out["8b_mixed_64_decodes_512_portion_ms"] = round(mms, 3)
            out["8b_mixed_tok_s"] = round(576 / (mms / 1e3), 1)
            read = z["weight_bytes"] + (64 * ctx + 1024 + 512) * z["kv_token_bytes"]
            flops = 2 * 576 * z["L"] * z["layer_params"] + 2 * 64 * z["V"] * z["H"]
            bound = max(read / (pk["hbm_gbs"] * 1e9), flops / (pk["bf16_tflops"] * 1e12))
            out["8b_mixed_frac_of_slower_bound"] = round(bound / (mms / 1e3), 4)
            # (both bounds: the decoded tokens' attention streams the cache while the tensor cores idle, the products
            # of 576 rows keep the tensor cores busy while little streams, and a layer runs them one after the other)
            out["8b_mixed_hbm_bound_ms"] = round(read / (pk["hbm_gbs"] * 1e9) * 1e3, 3)
            out["8b_mixed_flop_bound_ms"] = round(flops / (pk["bf16_tflops"] * 1e12) * 1e3, 3)
        del eng, runner
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
        gc.collect()
        torch.cuda.empty_cache()
    return out


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
        graph.replay()
    torch.cuda.synchronize()
    read()
    graph.replay()
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


def plain_cpu_baseline() -> int:
    """Seconds the plain float32 implementation under tests/ takes on the CPU for one whole-sequence forward
    pass of 64 tokens (it has no cache: every generated token costs such a pass): the timed CPU baseline of
    the tiny configurations and of the 0.6B shape."""
    import numpy as np
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_qwen3 as P
    from tiny_configs import TINY_A, TINY_B
    from paged_llm_rs_b200 import write_random_model

    out = {"what": "plain float32 implementation on the CPU, one forward pass of 64 tokens, best of 3",
           "threads": torch.get_num_threads()}
    tmp = tempfile.mkdtemp(prefix="pllm_plain_")
    try:
        for name, cfg in (("tiny_a", TINY_A), ("tiny_b", TINY_B), ("qwen3_0.6b_shape", SHAPE_0_6B)):
            d = write_random_model(os.path.join(tmp, name), cfg, 0)
            c, w = P.load_model(d, torch.float32)
            toks = np.random.default_rng(0).integers(0, cfg["vocab_size"], 64).tolist()
            best = 1e9
            for _ in range(3):
                t0 = time.time()
                with torch.no_grad():
                    P.forward(c, w, toks, rows=[63])
                best = min(best, time.time() - t0)
            out[name + "_s"] = round(best, 4)
            out[name + "_tok_s_prefill"] = round(64 / best, 1)
            out[name + "_tok_s_decode"] = round(1 / best, 2)
            del w
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    print(json.dumps(out))
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
    ap.add_argument("--no-shapes", action="store_true", help="skip the 8B and 32B shapes and the reference's kernel")
    ap.add_argument("--timeline-prefill", action="store_true",
                    help="with --only timeline: the captured step of a 2048-token prompt portion instead of the decode step")
    ap.add_argument("--timeline-mixed", type=int, default=0, metavar="TOKENS",
                    help="with --only timeline: the decoding requests beside one prompt portion of this many tokens")
    ap.add_argument("--only", choices=["decode", "prefill", "long-prompt", "timeline", "reference-kernel", "plain-cpu"], default=None,
                    help="run one part alone and print a short line (for profiling; not a bench record); "
                         "long-prompt: a prompt of --context tokens in portions of 2048, each portion timed; "
                         "timeline: one captured decode step as the kernels themselves clocked it; reference-kernel: "
                         "the reference's CUDA kernel against this engine's decode attention; plain-cpu: the plain "
                         "float32 implementation timed on the CPU (needs no GPU)")
    args = ap.parse_args(argv)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "nicoNaeg/paged-llm-rs is a Rust workspace (cargo, candle): pip cannot install it "
                          "('neither setup.py nor pyproject.toml found') and this image has no cargo or rustc"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.only == "plain-cpu":
        return plain_cpu_baseline()
    steps, warmup = args.steps, max(3, args.warmup)
    if args.only == "timeline":
        # a build of the kernels that stamps the global timer around each kernel's wait for its predecessor
        os.environ["PAGED_LLM_NVCC_DEFINES"] = (os.environ.get("PAGED_LLM_NVCC_DEFINES", "") + " PLLM_TRACE=1").strip()

    import gc
    import numpy as np
    import torch
    from paged_llm_rs_b200 import Engine, write_random_model

    pk = peaks()
    clocks = ClockSampler()
    if args.only == "reference-kernel":
        clocks.start()
        out = reference_kernel_points(clocks)
        out["clocks"] = clocks.stop()
        print(json.dumps(out))
        return 0
    shape_name, shape = SHAPES[args.shape][0], dict(SHAPES[args.shape][1])
    layers_full = shape["num_hidden_layers"]
    if args.layers:
        shape["num_hidden_layers"] = args.layers
    B, ctx = args.batch, args.context
    tmp = tempfile.mkdtemp(prefix="pllm_bench_", dir=scratch_dir())
    try:
        model_dir = write_random_model(os.path.join(tmp, "model"), shape, 0, device="cuda")
        most = 1 if (args.no_points or args.only) else 64
        pages = max(most, B) * (ctx // PAGE + 4) + PREFILL_TOKENS // PAGE + 64
        if args.only == "long-prompt":
            pages = ctx // PAGE + 64
        eng = Engine(model_dir, dtype="bfloat16", block_size=PAGE, blocks=pages, max_batch=max(most, B),
                     chunk=PREFILL_TOKENS, prefix_cache=False)
        runner = eng.runner
        for g in runner.cache.groups:       # cache contents for the device-timed points: random, not zeros
            g.pool.normal_(0.0, 1.0)
        z = shape_sizes(shape)
        L, H, I, nh, nkv, hd, V = z["L"], z["H"], z["I"], z["nh"], z["nkv"], z["hd"], z["V"]
        weight_bytes, kv_token_bytes = z["weight_bytes"], runner.cache.bytes_per_token()
        assert kv_token_bytes == z["kv_token_bytes"]
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

        if args.only == "long-prompt":
            out = long_prompt_points(runner, z, max(PREFILL_TOKENS, ctx // PREFILL_TOKENS * PREFILL_TOKENS), clocks)
            out.update(only="long-prompt", shape=shape_name, layers=L, clocks=clocks.stop())
            print(json.dumps(out))
            return 0

        if args.only == "timeline":
            return timeline(runner, B, ctx, L, PREFILL_TOKENS if args.timeline_prefill else 0, V, args.timeline_mixed)

        # -- decode, on the device -------------------------------------------------------
        ms, launches, spread = decode_point(runner, B, ctx, steps, warmup, clocks)
        if args.only == "decode":
            print(json.dumps({"only": "decode", "batch": B, "context": ctx, "ms_per_step": round(ms, 4),
                              "launches_per_step": launches, "repeats": spread}))
            return 0
        value = B / (ms / 1e3)
        step_bytes = weight_bytes + B * ctx * kv_token_bytes
        achieved = step_bytes / (ms / 1e3) / 1e9
        points = {}
        if not args.no_points:
            for c in (ctx, 512):                 # the bench context, and right after the baseline's 512-token prompts
                for b in (1, 8, 64):
                    if c == ctx and b == B:
                        continue
                    _, _, sp = decode_point(runner, b, c, max(10, steps // 2), warmup, clocks, repeats=4)
                    tag = f"decode_b{b}" + ("" if c == ctx else f"_ctx{c}")
                    points[tag] = round(b / (sp["median_ms"] / 1e3), 1)
                    points[tag + "_hbm_frac"] = round((weight_bytes + b * c * kv_token_bytes) / (sp["median_ms"] / 1e3) / 1e9
                                                      / pk["hbm_gbs"], 4)

        # -- prefill of 2048 tokens ---------------------------------------------------------
        pms, pspread = prefill_point(runner, V, clocks)
        prefill_out = dict(value=round(PREFILL_TOKENS / (pms / 1e3), 1), tokens=PREFILL_TOKENS, ms=round(pms, 3),
                           frac=round(z["prefill_flops"] / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                           frac_sustained=round(z["prefill_flops"] / (pms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
                           min_ms=pspread["min_ms"], max_ms=pspread["max_ms"], n=pspread["n"])

        # -- end to end through the entry point ---------------------------------------------
        rng = np.random.default_rng(1)
        rounds = 5
        budget = warmup + rounds * steps + 2
        for _ in range(B):
            eng.submit(rng.integers(0, V, ctx - budget - 16).tolist(), max_tokens=100000)
        while eng.scheduler.waiting or any(s.prompt_left for s in eng.scheduler.running):
            eng.step()                               # the prompts, untimed
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        per = []
        # (the prompts end so that the LAST round's steps run at the last positions before the bench's context, and
        #  that round is the one reported: the rounds before it, a little shorter in context, give the spread; a
        #  round past the context would need wider block tables and a capture of its own)
        for k in range(rounds):
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
            per.append((t1 - t0) / steps * 1e3)
            if k == rounds - 1:
                e2e = dict(value=round(B * steps / (t1 - t0), 1), unit="tokens/s", h2d_bytes_per_step=h2d // steps,
                           d2h_bytes_per_step=d2h // steps, ms_per_step=round((t1 - t0) / steps * 1e3, 4))
        e2e.update(n=rounds, median_ms=round(statistics.median(per), 4), min_ms=round(min(per), 4), max_ms=round(max(per), 4))
        del eng, runner
        gc.collect()
        torch.cuda.empty_cache()

        # -- whole generations: 64 requests from their prompts to their last token ---------------
        generate_out = {}
        if not args.no_points:
            try:
                generate_out = generate_point(model_dir, V, clocks)
            except Exception as e:     # noqa: BLE001
                generate_out = {"error": f"{type(e).__name__}: {e}"[:200]}
            gc.collect()
            torch.cuda.empty_cache()
        shutil.rmtree(tmp, ignore_errors=True)

        # -- the baseline's other shapes, and the reference's own kernel -------------------------------
        shapes, ref_kernel = {}, {}
        if not args.no_shapes and args.shape == "0.6b" and not args.layers:
            # (what fails here is written into its own block: the headline above is measured already)
            for key, layers_of in (("8b", None), ("32b", 16)):
                # 16 of the 32B shape's 64 layers: the whole model's 65 GB of random weights take minutes to draw
                # and load; the layers are the shape's own size
                try:
                    shapes.update(other_shape(key, layers_of, pk, clocks, steps, warmup))
                except Exception as e:     # noqa: BLE001
                    shapes[f"{key}_error"] = f"{type(e).__name__}: {e}"[:200]
                    gc.collect()
                    torch.cuda.empty_cache()
            try:
                ref_kernel = reference_kernel_points(clocks, reps=5)
            except Exception as e:     # noqa: BLE001
                ref_kernel = {"error": f"{type(e).__name__}: {e}"[:200]}
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
            "bf16_tflops_sustained": pk["bf16_tflops_sustained"],
        },
        "repeats": spread,
        "e2e": e2e, "gpu_launches": launches * steps, "clocks": clk, "prefill": prefill_out,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    if generate_out:
        line["generate"] = generate_out
    if shapes:
        line["shapes"] = shapes
    if ref_kernel:
        line["reference_kernel"] = ref_kernel
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
