"""Whole-model correctness at the layer sizes the bench runs: two layers of the
Qwen3-0.6B shape (hidden 1024, 16 query heads over 8 kv heads of 128, intermediate
3072, vocabulary 151 936, tied head) with random weights, in bfloat16 and in float32,
against the plain implementation in float64: a prompt of 2048 tokens as one captured
portion step, and eight requests decoding at contexts around 4096 through the captured
decode step, their prompts fed in portions of 2048."""

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu

SHAPE = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu", attention_bias=False,
    hidden_size=1024, intermediate_size=3072, num_hidden_layers=2, num_attention_heads=16, num_key_value_heads=8,
    head_dim=128, rms_norm_eps=1e-6, vocab_size=151936, max_position_embeddings=40960, tie_word_embeddings=True,
    rope_theta=1000000.0, sliding_window=None, use_sliding_window=False,
)
TOL = {"float32": 2e-5, "bfloat16": 3e-2}


def err(got, want):
    return float(np.abs(got - want).max() / max(1.0, np.abs(want).max()))


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    from paged_llm_rs_b200.weights.random_init import write_random_model

    d = str(tmp_path_factory.mktemp("real") / "two_layers_of_0_6b")
    write_random_model(d, SHAPE, 0, device="cuda")
    cfg, w = P.load_model(d, torch.float64, device="cuda")       # the plain functions, on the weights' device
    return d, cfg, w


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_two_layers_of_the_0_6b_shape_against_the_plain_implementation(model, dtype):
    from paged_llm_rs_b200.engine.runner import ModelRunner
    from paged_llm_rs_b200.engine.step import StepEntry

    d, cfg, w = model
    V = SHAPE["vocab_size"]
    rng = np.random.default_rng(3)
    runner = ModelRunner(d, dtype=dtype, page_size=16, num_pages=8 * 260 + 160, max_requests=16, prefix_cache=False)
    runner.graph_step_tokens = 2048
    cache = runner.cache
    zero1 = np.zeros(1, dtype=np.float32)

    # -- one prompt of 2048 tokens, whole: as a captured portion step, and launched with more rows wanted
    prompt = rng.integers(0, V, 2048).tolist()
    rows = list(range(0, 2048, 97)) + [2046, 2047]
    want = P.forward(cfg, w, prompt, rows=rows).cpu().numpy()
    cache.open("p")
    assert cache.reserve("p", 2048)
    logits, tokens = runner.step_and_sample([StepEntry("p", prompt, [2047])], zero1, zero1)
    assert runner._portion_graph([StepEntry("p", prompt, [2047])]) is not None      # it ran as a captured step
    got_last, tok = logits.cpu().numpy(), tokens.cpu().numpy()
    runner.check_status()
    assert err(got_last, want[-1:]) <= TOL[dtype]
    assert tok[1] == got_last[0].argmax()
    got = runner.step([StepEntry("p", prompt, rows)]).cpu().numpy()                   # the same tokens again, launched
    assert err(got, want) <= TOL[dtype]
    if dtype == "float32":
        assert (got.argmax(1) == want.argmax(1)).all() and got_last[0].argmax() == want[-1].argmax()
    cache.close("p")

    # -- eight requests decoding at contexts around 4096, fed tokens, through the captured decode step
    steps = 3
    ctx = [4096 - steps - 5 * i for i in range(8)]                    # tokens in the cache before the first decode step
    toks = [rng.integers(0, V, c + steps).tolist() for c in ctx]
    for r, c in enumerate(ctx):
        cache.open(r)
        for a in range(0, c, 2048):
            part = toks[r][a:min(a + 2048, c)]
            assert cache.reserve(r, len(part))
            runner.step_and_sample([StepEntry(r, part, [])], zero1[:0], zero1[:0])
            cache.commit(r, len(part))
    zeros = np.zeros(8, dtype=np.float32)
    got = []
    for i in range(steps):
        entries = [StepEntry(r, [toks[r][ctx[r] + i]], [0]) for r in range(8)]
        for r in range(8):
            assert cache.reserve(r, 1)
        logits, _ = runner.step_and_sample(entries, zeros, zeros)
        got.append(logits.cpu().numpy())
        for r in range(8):
            cache.commit(r, 1)
    runner.check_status()
    assert (8, 256) in runner._graphs                                 # the captured step of eight ran
    for r in range(8):
        want = P.forward(cfg, w, toks[r], rows=[ctx[r] + i for i in range(steps)]).cpu().numpy()
        have = np.stack([got[i][r] for i in range(steps)])
        assert err(have, want) <= TOL[dtype], r
        if dtype == "float32":
            assert (have.argmax(1) == want.argmax(1)).all(), r
        cache.close(r)
    cache.check_invariants()
