"""The engine itself on the reference's committed fixture: the tiny model the
reference's own tests load (crates/pagedllm/tests/fixtures/tiny, copied byte for
byte to tests/golden/reference_fixture) and the logits its dump holds for the
prompt of the manifest.  What the reference checks of its model
(crates/pagedllm/tests/forward.rs:53-79: logits within the manifest's tolerance
and equal argmax; crates/pagedllm/tests/batching.rs:185-205, 265-319: one token
at a time and in slices of 1, 3, 4 and 7 tokens equals one pass) is checked here
of this engine, through its step function, cache manager and kernels."""

import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

FIXTURE = os.path.join(os.path.dirname(__file__), "golden", "reference_fixture")


def fixture_logits():
    from safetensors.numpy import load_file

    manifest = json.load(open(os.path.join(FIXTURE, "manifest.json")))
    acts = load_file(os.path.join(FIXTURE, "activations.safetensors"))
    prompt = manifest["prompt"]
    return manifest, prompt, acts["logits"].reshape(len(prompt), -1).astype(np.float64), acts


def err(got, want):
    return float(np.abs(got - want).max() / max(1.0, np.abs(want).max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [4, 16])
def test_engine_reproduces_the_reference_dump_under_every_cut(dtype, page_size):
    from paged_llm_rs_b200.engine.runner import ModelRunner
    from paged_llm_rs_b200.engine.step import StepEntry

    manifest, prompt, want, _ = fixture_logits()
    tol = manifest["relative_tolerance"] if dtype == "float32" else 3e-2
    runner = ModelRunner(FIXTURE, dtype=dtype, page_size=page_size, num_pages=16, max_requests=4, prefix_cache=False)
    cache = runner.cache
    n = len(prompt)
    for size in (n, 1, 3, 4, 7):            # whole; token by token; the reference's slices
        rid = f"slices of {size}"
        cache.open(rid)
        got = []
        for a in range(0, n, size):
            part = prompt[a:a + size]
            assert cache.reserve(rid, len(part))
            got.append(runner.step([StepEntry(rid, part, list(range(len(part))))]).cpu().numpy())
            cache.commit(rid, len(part))
        got = np.concatenate(got)
        assert got.shape == want.shape
        assert err(got, want) <= tol, (size, err(got, want))
        if dtype == "float32":
            assert (got.argmax(1) == want.argmax(1)).all(), size
        cache.close(rid)
    # middle slices may ask for nothing and then get nothing (batching.rs:299-319)
    cache.open("quiet")
    assert cache.reserve("quiet", n)
    assert runner.step([StepEntry("quiet", prompt[:5], [])]).shape == (0, want.shape[1])
    cache.commit("quiet", 5)
    last = runner.step([StepEntry("quiet", prompt[5:], [n - 6])]).cpu().numpy()
    assert err(last, want[-1:]) <= tol
    cache.close("quiet")
    cache.check_invariants()


def test_engine_activations_by_module_name_match_the_reference_dump():
    """The reference compares 36 named tensors of its model with the dump
    (crates/pagedllm/tests/forward.rs:23-51, captured by crates/pagedllm/src/model/mod.rs:33-80).
    The engine records, under the same names, what its kernels leave at module
    boundaries in float32 (fused kernels leave fewer: what is never stored cannot be named)."""
    from paged_llm_rs_b200.engine.runner import ModelRunner
    from paged_llm_rs_b200.engine.step import StepEntry

    manifest, prompt, want, acts = fixture_logits()
    runner = ModelRunner(FIXTURE, dtype="float32", page_size=4, num_pages=8, max_requests=2, prefix_cache=False)
    runner.cache.open("t")
    assert runner.cache.reserve("t", len(prompt))
    trace = {}
    logits = runner.step([StepEntry("t", prompt, list(range(len(prompt))))], trace=trace)
    assert err(logits.cpu().numpy(), want) <= manifest["relative_tolerance"]
    names = set(manifest["tensors"])
    assert set(trace) <= names, sorted(set(trace) - names)
    must = {"model.embed_tokens.out", "model.norm.out", "logits", "lm_head.out"}
    for layer in range(manifest["num_hidden_layers"]):
        p = f"model.layers.{layer}"
        must |= {f"{p}.input_layernorm.out", f"{p}.self_attn.q_proj.out", f"{p}.self_attn.k_proj.out",
                 f"{p}.self_attn.v_proj.out", f"{p}.self_attn.o_proj.in", f"{p}.self_attn.o_proj.out", f"{p}.self_attn.out",
                 f"{p}.post_attention_layernorm.out", f"{p}.mlp.down_proj.in", f"{p}.mlp.down_proj.out", f"{p}.mlp.out", f"{p}.out"}
    assert must <= set(trace), sorted(must - set(trace))
    for name, got in trace.items():
        ref = acts[name]
        got = got.cpu().numpy()
        assert got.size == ref.size, name
        assert err(got.reshape(-1), ref.reshape(-1).astype(np.float64)) <= manifest["relative_tolerance"], name
