"""Weights: the container, the one error that lists everything wrong, roles and
dtypes, and the random-weights mode."""

import json
import os

import pytest
import torch

from paged_llm_rs_b200 import WeightError, write_random_model
from paged_llm_rs_b200.config import Qwen3Config
from paged_llm_rs_b200.models.qwen3 import describe_qwen3
from paged_llm_rs_b200.parts.decoder import tensor_specs_of
from paged_llm_rs_b200.weights import SafetensorsFile, check_tensors, load_weights, write_safetensors
from tiny_configs import TINY_A, TINY_B


def specs(cfg):
    return tensor_specs_of(describe_qwen3(Qwen3Config.from_dict(cfg)))


def test_container_round_trip_and_library_agrees(tmp_path):
    from safetensors.torch import load_file

    t = {"a.weight": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int32),
         "c": torch.randn(2, 2, 2), "empty": torch.zeros(0, 4)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t)
    f = SafetensorsFile(p)
    assert sorted(f.names()) == sorted(t)
    for k, v in t.items():
        assert f.dtype(k) == v.dtype and f.shape(k) == tuple(v.shape) and torch.equal(f.tensor(k), v)
    lib = load_file(p)
    assert all(torch.equal(lib[k], v) for k, v in t.items())


def test_truncated_file_is_refused(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x10\x00\x00")
    with pytest.raises(WeightError):
        SafetensorsFile(str(p))
    p.write_bytes((1000).to_bytes(8, "little") + b"{}")
    with pytest.raises(WeightError):
        SafetensorsFile(str(p))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, 0)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    t = {n: f.tensor(n).clone() for n in f.names()}
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63).bfloat16()
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        load_weights(d, specs(TINY_A), torch.float32, "cpu")
    msg = str(e.value)
    assert "missing (2)" in msg and "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected (1)" in msg and "rotary_emb.inv_freq" in msg
    assert "wrong shape (1)" in msg and "q_proj.weight has shape [64, 63], expected [64, 64]" in msg


def test_head_count_mismatch_shows_as_shape_error(tmp_path):
    # crates/pagedllm/tests/forward.rs:81-92: a config with other head counts than the file
    d = write_random_model(str(tmp_path / "m"), TINY_A, 0)
    with pytest.raises(WeightError, match="wrong shape"):
        load_weights(d, specs(dict(TINY_A, num_attention_heads=8, num_key_value_heads=4)), torch.float32, "cpu")


def test_untied_head_must_be_in_the_file(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, 0)  # tied: the file has no lm_head.weight
    names = SafetensorsFile(os.path.join(d, "model.safetensors")).names()
    assert "lm_head.weight" not in names
    load_weights(d, specs(TINY_A), torch.float32, "cpu")
    with pytest.raises(WeightError, match="missing.*lm_head.weight"):
        load_weights(d, specs(dict(TINY_A, tie_word_embeddings=False)), torch.float32, "cpu")


def test_roles_decide_dtypes(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_B, 1)
    for compute in (torch.bfloat16, torch.float32):
        w = load_weights(d, specs(TINY_B), compute, "cpu")
        assert w["model.layers.0.mlp.down_proj.weight"].dtype == compute   # matrices: compute dtype
        assert w["model.layers.0.input_layernorm.weight"].dtype == torch.float32  # gains: always float32
        assert w["lm_head.weight"].shape == (384, 96)
    # "keep": a tensor stored in 32-bit stays so; "index": int32
    from paged_llm_rs_b200.parts.spec import TensorSpec
    write_safetensors(os.path.join(d, "model.safetensors"),
                      {"s": torch.ones(4, dtype=torch.float32), "h": torch.ones(4).bfloat16(),
                       "i": torch.arange(4, dtype=torch.int64)})
    w = load_weights(d, [TensorSpec("s", (4,), "keep"), TensorSpec("h", (4,), "keep"), TensorSpec("i", (4,), "index")],
                     torch.bfloat16, "cpu")
    assert (w["s"].dtype, w["h"].dtype, w["i"].dtype) == (torch.float32, torch.bfloat16, torch.int32)


def test_random_weights_are_seeded_and_shaped(tmp_path):
    a = write_random_model(str(tmp_path / "a"), TINY_A, 0)
    b = write_random_model(str(tmp_path / "b"), TINY_A, 0)
    c = write_random_model(str(tmp_path / "c"), TINY_A, 1)
    read = lambda d: open(os.path.join(d, "model.safetensors"), "rb").read()
    assert read(a) == read(b) and read(a) != read(c)
    assert json.load(open(os.path.join(a, "config.json")))["hidden_size"] == 64
    f = SafetensorsFile(os.path.join(a, "model.safetensors"))
    m = f.tensor("model.layers.0.mlp.gate_proj.weight").float()
    g = f.tensor("model.layers.1.self_attn.q_norm.weight").float()
    assert f.dtype("model.embed_tokens.weight") == torch.bfloat16
    assert abs(m.std().item() - 0.02) < 0.002 and abs(m.mean().item()) < 0.002   # N(0, 0.02)
    assert abs(g.mean().item() - 1.0) < 0.1 and g.shape == (16,)                  # 1 + N(0, 0.1)


def test_sharded_checkpoint(tmp_path):
    d = write_random_model(str(tmp_path / "m"), TINY_A, 0)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    names = f.names()
    half = len(names) // 2
    parts = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    for fn, ns in parts.items():
        write_safetensors(os.path.join(d, fn), {n: f.tensor(n).clone() for n in ns})
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as out:
        json.dump({"weight_map": {n: fn for fn, ns in parts.items() for n in ns}}, out)
    whole = load_weights(d, specs(TINY_A), torch.float32, "cpu")
    os.remove(os.path.join(d, "model.safetensors"))
    sharded = load_weights(d, specs(TINY_A), torch.float32, "cpu")
    assert all(torch.equal(whole[k], sharded[k]) for k in whole)


@pytest.mark.gpu
def test_random_weights_do_not_depend_on_the_device_they_are_drawn_on(tmp_path):
    # every value is a function of (seed, tensor name, index) computed in integers: a folder written on the
    # GPU (the bench) holds the bytes of one written on the CPU (the tests)
    a = write_random_model(str(tmp_path / "cpu"), TINY_B, 5, device="cpu")
    b = write_random_model(str(tmp_path / "gpu"), TINY_B, 5, device="cuda")
    with open(a + "/model.safetensors", "rb") as f, open(b + "/model.safetensors", "rb") as g:
        assert f.read() == g.read()
