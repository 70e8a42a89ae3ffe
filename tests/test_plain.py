"""The plain implementation against the reference's committed fixture, and its
small parts against hand-checked values."""

import json
import math
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as P

FIXTURE = os.path.join(os.path.dirname(__file__), "golden", "reference_fixture")


def test_plain_matches_reference_fixture():
    # crates/pagedllm/tests/forward.rs:23-51: every dumped tensor within the manifest's
    # tolerance, measured as worst |got - want| / max(1, max |want|), and equal argmax.
    from safetensors.torch import load_file

    cfg, w = P.load_model(FIXTURE)
    manifest = json.load(open(os.path.join(FIXTURE, "manifest.json")))
    acts = load_file(os.path.join(FIXTURE, "activations.safetensors"))
    trace = {}
    logits = P.forward(cfg, w, manifest["prompt"], trace)
    assert len(manifest["tensors"]) == 36
    for name in manifest["tensors"]:
        got, want = trace[name], acts[name]
        assert got.numel() == want.numel(), name
        want = want.reshape(got.shape)
        err = (got - want).abs().max().item() / max(1.0, want.abs().max().item())
        assert err <= manifest["relative_tolerance"], (name, err)
    assert logits.argmax(-1).tolist() == acts["logits"].reshape(logits.shape).argmax(-1).tolist()


def test_rope_position_zero_is_identity_and_pairs_halves():
    cos, sin = P.rope_tables(8, 4, 10000.0)
    x = torch.arange(8, dtype=torch.float32).reshape(1, 1, 8)
    assert torch.equal(P.apply_rope(x, cos[:1], sin[:1]), x)
    # dimension i pairs with i + 4: rotating (1, 0) in the pair (0, 4) by angle 1 at position 1
    e = torch.zeros(1, 1, 8)
    e[0, 0, 0] = 1.0
    y = P.apply_rope(e, cos[1:2], sin[1:2])
    assert y[0, 0, 0].item() == pytest.approx(math.cos(1.0), abs=1e-6)
    assert y[0, 0, 4].item() == pytest.approx(math.sin(1.0), abs=1e-6)
    assert P.rotate_half(torch.tensor([1.0, 2.0, 3.0, 4.0])).tolist() == [-3.0, -4.0, 1.0, 2.0]


def test_rms_norm_eps_inside_root():
    x = torch.tensor([[3.0, 4.0]])
    y = P.rms_norm(x, torch.tensor([1.0, 2.0]), 0.5)
    r = math.sqrt(12.5 + 0.5)
    assert y.tolist()[0] == pytest.approx([3.0 / r, 8.0 / r])


def test_causal_mask_and_window():
    m = P.causal_mask(4, None, torch.float32)
    assert (m == 0).sum().item() == 10 and m[1, 2] == float("-inf") and m[2, 2] == 0
    w = P.causal_mask(5, 2, torch.float32)  # sees itself and one key before
    assert [(w[4] == 0).nonzero().flatten().tolist()] == [[3, 4]]


def test_splitmix_and_greedy():
    r = P.PlainRng(0)
    assert r.next_u64() == 0xE220A8397B1DCDAF  # splitmix64's first output for seed 0
    assert 0.0 <= P.PlainRng(7).next_f32() < 1.0
    assert P.greedy(torch.tensor([1.0, 3.0, 3.0, 2.0])) == 1  # the first maximum


def test_sampler_distribution_and_top_k_top_p():
    logits = torch.log(torch.tensor([0.5, 0.3, 0.15, 0.05]))
    rng = P.PlainRng(1)
    counts = np.zeros(4)
    for _ in range(20000):
        counts[P.sample(logits, 1.0, None, None, rng)] += 1
    assert np.abs(counts / 20000 - np.array([0.5, 0.3, 0.15, 0.05])).max() < 0.012
    assert all(P.sample(logits, 1.0, 1, None, P.PlainRng(s)) == 0 for s in range(20))
    # top_p 0.7: 0.5 does not reach it, 0.5 + 0.3 crosses and is kept; nothing else is
    assert {P.sample(logits, 1.0, None, 0.7, P.PlainRng(s)) for s in range(200)} == {0, 1}


@pytest.mark.parametrize("name", ["A", "D"])
def test_the_models_for_checks_on_tokens_let_attention_decide(tmp_path, name):
    """Checks on generated tokens use folders drawn wider than N(0, 0.02) and with a head of their
    own (tiny_configs.write_model(..., decisive=True)): there the next token changes when the
    attention output is zeroed, and the model does not simply repeat its last token.  With
    N(0, 0.02) and a tied head neither holds often enough for a token to say much about the cache."""
    from tiny_configs import CONFIGS, write_model

    cfg, seed = CONFIGS[name]
    model = write_model(tmp_path, name, decisive=True)
    c, w = P.load_model(model, torch.float64)
    silent = {k: (v * 0 if "o_proj" in k else v) for k, v in w.items()}
    rng = np.random.default_rng(9)
    moved = echoes = total = 0
    for n in (7, 19, 40):
        seq = rng.integers(0, cfg["vocab_size"], n).tolist()
        for _ in range(8):
            a = int(P.forward(c, w, seq)[-1].argmax())
            moved += a != int(P.forward(c, silent, seq)[-1].argmax())
            echoes += a == seq[-1]
            total += 1
            seq.append(a)
    assert moved >= 0.9 * total and echoes <= 0.5 * total, (moved, echoes, total)
