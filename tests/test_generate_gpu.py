"""Generation through the Python entry point against the plain implementation:
greedy (identical tokens in float32), temperature draws, top-k / top-p, a shared
prefix, preemption in a pool that is too small, and the command line."""

import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from tiny_configs import CONFIGS, write_model

pytestmark = pytest.mark.gpu


def prompts_for(vocab, lengths, seed, shared=0):
    rng = np.random.default_rng(seed)
    ps = [rng.integers(0, vocab, n).tolist() for n in lengths]
    if shared:
        ps[-1][:shared] = ps[-2][:shared]
    return ps


def plain_greedy(model, prompt, n):
    cfg, w = P.load_model(model, torch.float64)
    seq, gaps = list(prompt), []
    for _ in range(n):
        logits = P.forward(cfg, w, seq)[-1]
        top2 = torch.topk(logits, 2).values
        gaps.append(float(top2[0] - top2[1]))
        seq.append(P.greedy(logits))
    return seq[len(prompt):], gaps


# bfloat16 may choose another token only where the float64 decision was closer than its noise:
# this fraction of the largest logit (8 mantissa bits through a few layers; observed below 1e-2)
BF16_NOISE = 0.03


def check_greedy(model, prompts, outs, n, dtype, min_decided=0.5):
    """Every token the engine produced against the plain implementation run on the same
    history (the prompt and the engine's own tokens so far), so that a token that differs
    does not end the check.  float32: the plain argmax, everywhere.  bfloat16: the plain
    argmax wherever the plain decision is wider than bfloat16's noise, and elsewhere a
    token whose plain logit is within that noise of the largest."""
    cfg, w = P.load_model(model, torch.float64)
    decided = total = echoes = 0
    for p, o in zip(prompts, outs):
        assert len(o) == n
        seq = list(p)
        for i, tok in enumerate(o):
            logits = P.forward(cfg, w, seq)[-1]
            best = P.greedy(logits)
            if dtype == "float32":
                assert tok == best, (i, tok, best)
            else:
                noise = BF16_NOISE * max(1.0, float(logits.abs().max()))
                assert float(logits[best] - logits[tok]) < noise, (i, tok, best, float(logits[best] - logits[tok]), noise)
                top2 = torch.topk(logits, 2).values
                decided += float(top2[0] - top2[1]) >= noise
            echoes += tok == seq[-1]
            total += 1
            seq.append(tok)
    if dtype != "float32":
        assert decided >= min_decided * total, f"only {decided} of {total} decisions are wider than bfloat16's noise"
    return echoes, total


def attention_decides(model, prompts, n=4):
    """How often the plain implementation's next token changes when every attention output is
    zeroed: a model where it does not says nothing about the cache in a check on tokens."""
    cfg, w = P.load_model(model, torch.float64)
    silent = {k: (v * 0 if "o_proj" in k else v) for k, v in w.items()}
    moved = total = 0
    for p in prompts:
        seq = list(p)
        for _ in range(n):
            a, b = P.forward(cfg, w, seq)[-1], P.forward(cfg, silent, seq)[-1]
            moved += int(a.argmax()) != int(b.argmax())
            total += 1
            seq.append(int(a.argmax()))
    return moved, total


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_tiny_a(tmp_path, dtype):
    # three requests with prompts of 1, 7 and 19 tokens, 8 greedy tokens each, pages of 16, budget 8
    from paged_llm_rs_b200 import Engine
    cfg, seed = CONFIGS["A"]
    model = write_model(tmp_path, "A", decisive=True)
    prompts = prompts_for(cfg["vocab_size"], [1, 7, 19], 11)
    moved, total = attention_decides(model, prompts[1:])
    assert moved >= total - 1                       # (a prompt of one token has nothing to attend to but itself)
    eng = Engine(model, dtype=dtype, block_size=16, blocks=32, chunk=8)
    outs = eng.generate(prompts, max_tokens=8)
    echoes, total = check_greedy(model, prompts, outs, 8, dtype)
    assert echoes <= total // 2                     # not a model that repeats its last token
    m = eng.metrics()
    assert m["mixed_steps"] > 0 and m["tokens"] == 24 and m["pages_free"] == 32
    # whole prompts (chunk off) give the same tokens
    eng2 = Engine(model, dtype=dtype, block_size=16, blocks=32, chunk=None)
    assert eng2.generate(prompts, max_tokens=8) == outs or dtype == "bfloat16"
    # several prompts in one pass: fewer steps, and in float32 the same tokens
    eng3 = Engine(model, dtype=dtype, block_size=16, blocks=32, chunk=24, max_prefill_seqs=3)
    outs3 = eng3.generate(prompts, max_tokens=8)
    check_greedy(model, prompts, outs3, 8, dtype)
    assert outs3 == outs or dtype == "bfloat16"
    eng4 = Engine(model, dtype=dtype, block_size=16, blocks=32, chunk=24)
    eng4.generate(prompts, max_tokens=8)
    assert eng3.metrics()["steps"] < eng4.metrics()["steps"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_tiny_d_tensor_core_kernels(tmp_path, dtype):
    # head_dim 64: in bfloat16 the prompts run through the mma kernel, decoding through the
    # bulk-copy kernel over the swizzled cache, and decode steps replay as CUDA graphs
    from paged_llm_rs_b200 import Engine
    cfg, seed = CONFIGS["D"]
    model = write_model(tmp_path, "D", decisive=True)
    prompts = prompts_for(cfg["vocab_size"], [90, 3, 130, 64], 21)
    moved, total = attention_decides(model, prompts)
    assert moved >= total - 2
    eng = Engine(model, dtype=dtype, block_size=16, blocks=64, chunk=48)
    outs = eng.generate(prompts, max_tokens=24)
    echoes, total = check_greedy(model, prompts, outs, 24, dtype)
    assert echoes <= total // 2
    plain = Engine(model, dtype=dtype, block_size=16, blocks=64, chunk=48)
    plain.runner.use_graphs = False
    assert plain.generate(prompts, max_tokens=24) == outs          # captured and plain launches agree


def test_greedy_many_requests_decoding_beside_prompt_portions(tmp_path):
    # twelve requests under a token budget: from the ninth on, the decoded tokens of a mixed step run on the
    # bulk-copy kernel beside the tcgen05 kernel that takes the portion (two streams that meet again)
    from paged_llm_rs_b200 import Engine
    from paged_llm_rs_b200.kernels import ops
    cfg, seed = CONFIGS["D"]
    model = write_model(tmp_path, "D", decisive=True)
    prompts = prompts_for(cfg["vocab_size"], [70, 66, 90, 64, 130, 75, 68, 81, 99, 64, 72, 110], 23)
    assert ops.MIXED_BESIDE
    outs = {}
    for graphs in (True, False):
        eng = Engine(model, dtype="bfloat16", block_size=16, blocks=160, chunk=96, max_batch=16)
        eng.runner.use_graphs = graphs
        calls = ops.MIXED_BESIDE_CALLS
        outs[graphs] = eng.generate(prompts, max_tokens=40)
        check_greedy(model, prompts, outs[graphs], 40, "bfloat16")
        assert eng.metrics()["mixed_steps"] >= 10
        assert ops.MIXED_BESIDE_CALLS > calls          # (captured: once a layer at capture; plain: every such step)
    assert outs[True] == outs[False]


def test_warming_up_captures_the_steps_and_changes_no_token(tmp_path):
    # the steps captured ahead of time are the ones the requests then replay: no capture is made while they
    # run, and the tokens are those of an engine that captured as it went
    from paged_llm_rs_b200 import Engine
    cfg, seed = CONFIGS["D"]
    model = write_model(tmp_path, "D", decisive=True)
    prompts = prompts_for(cfg["vocab_size"], [70, 66, 90, 64, 130, 75], 31)
    cold = Engine(model, dtype="bfloat16", block_size=16, blocks=160, chunk=96, max_batch=8)
    want = cold.generate(prompts, max_tokens=24)
    warm = Engine(model, dtype="bfloat16", block_size=16, blocks=160, chunk=96, max_batch=8)
    made = warm.warm_up()
    assert made == 8 and warm.warm_up() == 0            # 1, 2, 4 and 8 requests: decode steps and the budget's steps
    held = len(warm.runner._graphs)
    assert warm.generate(prompts, max_tokens=24) == want
    assert len(warm.runner._graphs) == held
    check_greedy(model, prompts, want, 24, "bfloat16")


def vocab_order_choice(logits64, temperature, u):
    """The engine's device draw: ids upward, the first id whose running sum reaches u * total."""
    p = torch.softmax(logits64 / temperature, -1)
    cdf = torch.cumsum(p, 0)
    return cdf, float(u)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_tiny_b(tmp_path, dtype):
    # five requests, prompts of 3, 11, 24, 40 and 40 tokens (the last two share 32), 12 tokens at
    # temperature 0.8 with seed 7, pages of 8, budget 16: the last request takes the four pages
    # that hold the 32 tokens it shares with the one before it
    from paged_llm_rs_b200 import Engine
    cfg, seed = CONFIGS["B"]
    model = write_model(tmp_path, "B")
    prompts = prompts_for(cfg["vocab_size"], [3, 11, 24, 40, 40], 12, shared=32)
    eng = Engine(model, dtype=dtype, block_size=8, blocks=64, chunk=16)
    outs = eng.generate(prompts, max_tokens=12, temperature=0.8, seed=7)
    assert eng.metrics()["cached_tokens"] == 32
    assert outs == Engine(model, dtype=dtype, block_size=8, blocks=64, chunk=16).generate(
        prompts, max_tokens=12, temperature=0.8, seed=7)                      # the same seed, the same tokens
    c, w = P.load_model(model, torch.float64)
    slack = 1e-4 if dtype == "float32" else 2e-2
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        rng = P.PlainRng(7)
        for i, tok in enumerate(o):
            logits = P.forward(c, w, p + o[:i])[-1]
            cdf, u = vocab_order_choice(logits, 0.8, rng.next_f32())
            lo = float(cdf[tok - 1]) if tok > 0 else 0.0
            assert lo - slack <= u <= float(cdf[tok]) + slack, (i, tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_packing_the_next_step_ahead_changes_nothing(tmp_path, dtype):
    # the engine that gets the next decode step ready while the current one runs, against the one that
    # does not: the same tokens, endings and counters, with requests that end at different times (budgets,
    # a stop token), some of them drawing at a temperature, so few pages that one request is preempted,
    # and a request that arrives while the others decode
    from paged_llm_rs_b200 import Engine
    cfg, seed = CONFIGS["W"]
    model = write_model(tmp_path, "W")
    prompts = prompts_for(cfg["vocab_size"], [3, 11, 24, 40, 17], 31)
    budgets = [30, 9, 18, 25, 12]
    def run(ahead, blocks):
        eng = Engine(model, dtype=dtype, block_size=8, blocks=blocks, chunk=16, lookahead=ahead)
        ids = [eng.submit(p, max_tokens=b, temperature=0.0 if i % 2 else 0.8, seed=5 + i, stop_tokens=[7, 300])
               for i, (p, b) in enumerate(zip(prompts[:4], budgets))]
        outs, late, steps = {}, None, 0
        while eng.scheduler.has_work():
            out = eng.step()
            steps += 1
            assert out is not None
            for rid, tok in out.tokens:
                outs.setdefault(rid, []).append(tok)
            if steps == 12:
                late = eng.submit(prompts[4], max_tokens=budgets[4])
        assert eng._inflight is None
        m = eng.metrics()
        assert m["pages_free"] == blocks
        return (outs, {i: eng.finish_reason(i) for i in ids + [late]},
                {k: m[k] for k in ("steps", "tokens", "decode_rows", "decode_steps", "mixed_steps", "preemptions")})

    with_it, without = run(True, 22), run(False, 22)
    assert with_it == without and with_it[2]["decode_steps"] >= 10 and with_it[2]["preemptions"] == 0
    # a pool that cannot hold them all: who is preempted when may differ (the pages of the step after next are
    # taken a step earlier), what each request produces may not
    if dtype != "float32":
        return      # (a request recomputed at another time rounds differently in bfloat16: nothing to compare)
    with_it, without = run(True, 13), run(False, 13)
    assert with_it[:2] == without[:2]
    assert with_it[2]["preemptions"] >= 1 and without[2]["preemptions"] >= 1
    assert with_it[2]["tokens"] == without[2]["tokens"]


def test_cancel_while_the_next_step_already_runs(tmp_path):
    # a request is cancelled between two calls of step(), when the engine has a decode step with it in flight:
    # its pages go back at once, its token of that step is dropped, the others go on as if nothing had happened
    from paged_llm_rs_b200 import Engine
    from paged_llm_rs_b200.engine.scheduler import Finish
    cfg, seed = CONFIGS["A"]
    model = write_model(tmp_path, "A", decisive=True)
    prompts = prompts_for(cfg["vocab_size"], [5, 9, 12], 17)
    full = Engine(model, dtype="float32", block_size=16, blocks=32, chunk=8).generate(prompts, max_tokens=20)
    eng = Engine(model, dtype="float32", block_size=16, blocks=32, chunk=8)
    ids = [eng.submit(p, max_tokens=20) for p in prompts]
    outs, cancelled_at = {i: [] for i in ids}, None
    while eng.scheduler.has_work():
        out = eng.step()
        for rid, tok in out.tokens:
            outs[rid].append(tok)
        if cancelled_at is None and len(outs[ids[1]]) == 6:
            assert eng._inflight is not None and ids[1] in eng._inflight[0].ids     # the step after is on its way
            eng.cancel(ids[1])
            cancelled_at = len(outs[ids[1]])
    assert cancelled_at == 6 and outs[ids[1]] == full[1][:6]
    assert outs[ids[0]] == full[0] and outs[ids[2]] == full[2]
    assert eng._inflight is None and eng.metrics()["pages_free"] == 32
    assert eng.finish_reason(ids[0]) == Finish.LENGTH


def test_cancelling_every_request_leaves_no_step_in_flight(tmp_path):
    # both requests are cancelled while the decode step after the last collected one already runs: the engine
    # waits for that step, checks its status and drops its tokens, so nothing runs on when nobody is left,
    # and the next generation starts from a clean engine
    from paged_llm_rs_b200 import Engine
    cfg, seed = CONFIGS["A"]
    model = write_model(tmp_path, "A", decisive=True)
    prompts = prompts_for(cfg["vocab_size"], [5, 9], 18)
    eng = Engine(model, dtype="float32", block_size=16, blocks=32, chunk=8)
    want = Engine(model, dtype="float32", block_size=16, blocks=32, chunk=8).generate(prompts, max_tokens=10)
    ids = [eng.submit(p, max_tokens=50) for p in prompts]
    produced = 0
    while produced < 8:
        produced += len(eng.step().tokens)
    assert eng._inflight is not None
    eng.cancel(ids[0])
    assert eng._inflight is not None            # the other request still runs
    eng.cancel(ids[1])
    assert eng._inflight is None and not eng.scheduler.has_work() and eng.last_error is None
    assert eng.metrics()["pages_free"] == 32
    eng.runner.cache.check_invariants()
    assert eng.generate(prompts, max_tokens=10) == want


def test_top_k_top_p_follow_the_reference_order(tmp_path):
    from paged_llm_rs_b200 import Engine
    cfg, seed = CONFIGS["A"]
    model = write_model(tmp_path, "A")
    prompts = prompts_for(cfg["vocab_size"], [5, 9], 13)
    eng = Engine(model, dtype="float32", blocks=32)
    outs = eng.generate(prompts, max_tokens=10, temperature=0.9, top_k=20, top_p=0.9, seed=3)
    c, w = P.load_model(model, torch.float64)
    for p, o in zip(prompts, outs):
        rng = P.PlainRng(3)
        for i, tok in enumerate(o):
            logits = P.forward(c, w, p + o[:i])[-1].float()
            assert tok == P.sample(logits, 0.9, 20, 0.9, rng), i


def test_temperature_in_the_reference_order_when_asked(tmp_path):
    # the device draws by walking token ids upward; with reference_draw_order the host draws by falling
    # probability (crates/pagedllm/src/sampler.rs:143-183), which for a seed gives the reference's tokens
    from paged_llm_rs_b200 import Engine
    cfg, seed = CONFIGS["A"]
    model = write_model(tmp_path, "A")
    prompts = prompts_for(cfg["vocab_size"], [5, 9], 13)
    outs = Engine(model, dtype="float32", blocks=32, reference_draw_order=True).generate(
        prompts, max_tokens=10, temperature=0.9, seed=3)
    c, w = P.load_model(model, torch.float64)
    for p, o in zip(prompts, outs):
        rng = P.PlainRng(3)
        for i, tok in enumerate(o):
            logits = P.forward(c, w, p + o[:i])[-1].float()
            assert tok == P.sample(logits, 0.9, None, None, rng), i
    other = Engine(model, dtype="float32", blocks=32).generate(prompts, max_tokens=10, temperature=0.9, seed=3)
    assert other != outs         # (the device's order: other tokens for the same seed)


def test_shared_prefix_gives_the_same_tokens(tmp_path):
    # crates/pagedllm/tests/prefix.rs:88-139: shared equals computed
    from paged_llm_rs_b200 import Engine
    cfg, seed = CONFIGS["A"]
    model = write_model(tmp_path, "A", decisive=True)
    prompts = prompts_for(cfg["vocab_size"], [50, 50, 50], 14, shared=32)
    prompts[0][:32] = prompts[1][:32]
    on = Engine(model, dtype="float32", blocks=64, chunk=16, prefix_cache=True)
    off = Engine(model, dtype="float32", blocks=64, chunk=16, prefix_cache=False)
    a, b = on.generate(prompts, max_tokens=6), off.generate(prompts, max_tokens=6)
    assert a == b
    assert on.metrics()["cached_tokens"] == 64 and off.metrics()["cached_tokens"] == 0
    check_greedy(model, prompts, a, 6, "float32")


def test_preemption_changes_no_token(tmp_path):
    from paged_llm_rs_b200 import Engine
    cfg, seed = CONFIGS["A"]
    model = write_model(tmp_path, "A", decisive=True)
    prompts = prompts_for(cfg["vocab_size"], [20, 25, 18, 22], 15)
    big = Engine(model, dtype="float32", block_size=8, blocks=64, chunk=16, prefix_cache=False)
    small = Engine(model, dtype="float32", block_size=8, blocks=14, chunk=16, prefix_cache=False)
    a, b = big.generate(prompts, max_tokens=20), small.generate(prompts, max_tokens=20)
    assert small.metrics()["preemptions"] > 0 and big.metrics()["preemptions"] == 0
    assert a == b
    small.runner.cache.check_invariants()
    assert small.metrics()["pages_free"] == 14


def test_stop_tokens_and_refusal(tmp_path):
    from paged_llm_rs_b200 import Engine
    from paged_llm_rs_b200.engine.scheduler import Finish
    cfg, seed = CONFIGS["A"]
    model = write_model(tmp_path, "A", decisive=True)
    eng = Engine(model, dtype="float32", block_size=8, blocks=4)
    p = prompts_for(cfg["vocab_size"], [6], 16)[0]
    free = eng.generate([p], max_tokens=6)[0]
    stop = free[-1]
    stopped = eng.generate([p], max_tokens=6, stop_tokens=[stop])[0]
    assert stopped == free[:free.index(stop)]                    # the stop token ends it and is not returned
    rid = eng.submit(list(range(40)), max_tokens=4)              # 5 pages of 8 can never fit in 4
    eng.run_until_done()
    assert eng.finish_reason(rid) == Finish.LENGTH and eng._seqs[rid].output == []


def test_command_line(tmp_path):
    cfg, seed = CONFIGS["A"]
    model = write_model(tmp_path, "A", decisive=True)
    r = subprocess.run([sys.executable, "-m", "paged_llm_rs_b200", "generate", "--model", model, "--dtype", "f32",
                        "--prompt-ids", "5,6,7", "--prompt-ids", "9", "--max-tokens", "5", "--blocks", "16",
                        "--chunk", "off", "--prefix-cache", "off", "--metrics"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = r.stdout.strip().splitlines()
    assert len(lines) == 2 and all(len(l.split(",")) == 5 for l in lines)
    want, _ = plain_greedy(model, [5, 6, 7], 5)
    assert [int(t) for t in lines[0].split(",")] == want
