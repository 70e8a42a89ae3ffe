"""Configurations at sizes the other tests do not reach, each through trace replay (portions of
changing size, single tokens, two requests side by side) against the plain implementation, in
float32 and in bfloat16: head sizes 80, 112 and 256 (multiples of 16 that no tensor-core kernel of
this engine takes), a single head, a group of 7 query heads to a kv head, as many kv heads as heads,
a width of 104 (rows that are no multiple of 16 bytes wide times anything useful), an intermediate
size of 88 and vocabularies of 97 and 1001.  A size that a kernel does not take must be refused or
taken by another kernel; never a wrong result."""

import numpy as np
import pytest

from trace_tools import TraceBuilder, plain_logits, replay

pytestmark = pytest.mark.gpu

BASE = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu", rms_norm_eps=1e-6,
            max_position_embeddings=256, rope_theta=10000.0, tie_word_embeddings=True)
ODD = {
    "hd80_group1": dict(BASE, hidden_size=104, intermediate_size=88, num_hidden_layers=2, num_attention_heads=3,
                        num_key_value_heads=3, head_dim=80, vocab_size=97),
    "hd112_group7": dict(BASE, hidden_size=72, intermediate_size=200, num_hidden_layers=2, num_attention_heads=7,
                         num_key_value_heads=1, head_dim=112, vocab_size=1001, tie_word_embeddings=False),
    "hd256_one_head": dict(BASE, hidden_size=136, intermediate_size=264, num_hidden_layers=1, num_attention_heads=1,
                           num_key_value_heads=1, head_dim=256, vocab_size=300, rms_norm_eps=1e-5),
    "hd128_group3": dict(BASE, hidden_size=200, intermediate_size=328, num_hidden_layers=2, num_attention_heads=6,
                         num_key_value_heads=2, head_dim=128, vocab_size=515, rope_theta=1e6),
}
TOL = {"float32": 2e-5, "bfloat16": 3e-2}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ODD))
def test_odd_sizes_through_replay(tmp_path, name, dtype):
    import torch
    from paged_llm_rs_b200.weights.random_init import write_random_model

    cfg = ODD[name]
    model = write_random_model(str(tmp_path / name), cfg, 21, torch.bfloat16)
    vocab = cfg["vocab_size"]
    rng = np.random.default_rng(5)
    toks = {"a": rng.integers(0, vocab, 75).tolist(), "b": rng.integers(0, vocab, 41).tolist()}
    tb = TraceBuilder()
    tb.step([("a", toks["a"][:19], range(19))])
    tb.step([("a", toks["a"][19:21], range(2)), ("b", toks["b"][:33], range(33))])
    tb.step([("a", toks["a"][21:22], [0]), ("b", toks["b"][33:34], [0])])
    tb.step([("a", toks["a"][22:70], range(48)), ("b", toks["b"][34:35], [0])])
    for i in range(35, 41):
        tb.step([("b", [toks["b"][i]], [0]), ("a", [toks["a"][35 + i]], [0])] if i < 40 else [("b", [toks["b"][i]], [0])],
                end=["b"] if i == 40 else [])
    tb.step([], end=["a"])
    got = replay(model, dtype, tb.steps, 128, vocab, page_size=16)
    want = {r: plain_logits(model, t) for r, t in toks.items()}
    seen = 0
    for step, row, rid, pos in tb.where:
        w = want[rid][pos]
        err = np.abs(got[step][row] - w).max() / max(1.0, np.abs(want[rid]).max())
        assert err <= TOL[dtype], (name, dtype, rid, pos, err)
        seen += 1
    assert seen == 19 + 2 + 33 + 2 + 48 + 1 + 5 * 2 + 1
