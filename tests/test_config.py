"""Configuration and registry (crates/pagedllm/src/config.rs:233-324 has the
reference's cases: the published 0.6B shape, the nested rope layout, refusals)."""

import copy
import json

import pytest

from paged_llm_rs_b200 import (ConfigError, GenerationDefaults, Qwen3Config, UnsupportedModelError, load_config,
                               register_architecture, resolve_architecture)
from paged_llm_rs_b200.config import Architecture
from paged_llm_rs_b200.models.qwen3 import describe_qwen3
from tiny_configs import TINY_A, TINY_B, TINY_W

QWEN3_0_6B = dict(
    architectures=["Qwen3ForCausalLM"], attention_bias=False, attention_dropout=0.0, bos_token_id=151643,
    eos_token_id=151645, head_dim=128, hidden_act="silu", hidden_size=1024, initializer_range=0.02,
    intermediate_size=3072, max_position_embeddings=40960, max_window_layers=28, model_type="qwen3",
    num_attention_heads=16, num_hidden_layers=28, num_key_value_heads=8, rms_norm_eps=1e-06, rope_scaling=None,
    rope_theta=1000000, sliding_window=None, tie_word_embeddings=True, torch_dtype="bfloat16",
    use_cache=True, use_sliding_window=False, vocab_size=151936)


def test_published_shape_parses():
    c = Qwen3Config.from_dict(QWEN3_0_6B)
    assert (c.hidden_size, c.num_hidden_layers, c.head_dim, c.vocab_size) == (1024, 28, 128, 151936)
    assert c.kv_group_size == 2 and c.query_width == 2048 and c.kv_width == 1024
    assert c.rope_theta == 1e6 and c.tie_word_embeddings and c.sliding_window is None
    assert set(c.layer_types) == {"full_attention"}


def test_round_trip_and_both_tiny_configs():
    for d in (TINY_A, TINY_B, TINY_W):
        c = Qwen3Config.from_dict(d)
        assert Qwen3Config.from_dict(c.to_dict()) == c
    b = Qwen3Config.from_dict(TINY_B)
    assert b.rope_theta == 1e6  # nested under rope_parameters
    assert [b.window_of_layer(i) for i in range(3)] == [None, None, None]
    assert [Qwen3Config.from_dict(TINY_W).window_of_layer(i) for i in range(3)] == [40, None, 40]


@pytest.mark.parametrize("change,error", [
    (dict(model_type="llama"), UnsupportedModelError),
    (dict(hidden_act="gelu"), UnsupportedModelError),
    (dict(attention_bias=True), UnsupportedModelError),
    (dict(rope_scaling={"type": "yarn"}), UnsupportedModelError),
    (dict(rope_parameters={"rope_theta": 1e6, "rope_type": "yarn"}, rope_theta=None), UnsupportedModelError),
    (dict(sliding_window=4096), UnsupportedModelError),           # a window that is switched off is refused
    (dict(num_key_value_heads=3), UnsupportedModelError),         # 4 heads over 3 kv heads
    (dict(rope_theta=None), ConfigError),                         # neither layout
    (dict(head_dim=None), ConfigError),                           # its own key, no default
    (dict(rms_norm_eps="tiny"), ConfigError),
    (dict(vocab_size=-5), ConfigError),
    (dict(use_sliding_window=True), ConfigError),                 # switched on without a size
    (dict(layer_types=["full_attention"]), ConfigError),          # wrong count
    (dict(layer_types=["full_attention", "linear_attention"]), UnsupportedModelError),
])
def test_refusals(change, error):
    d = copy.deepcopy(TINY_A)
    d.update(change)
    with pytest.raises(error):
        Qwen3Config.from_dict(d)


def test_window_from_max_window_layers():
    d = dict(TINY_A, use_sliding_window=True, sliding_window=8, max_window_layers=1)
    c = Qwen3Config.from_dict(d)
    assert c.layer_types == ("full_attention", "sliding_attention") and c.sliding_window == 8


def test_registry(tmp_path):
    assert resolve_architecture(TINY_A).name == "Qwen3ForCausalLM"
    assert resolve_architecture({"model_type": "qwen3"}).name == "Qwen3ForCausalLM"
    with pytest.raises(UnsupportedModelError, match="Mamba"):
        resolve_architecture({"architectures": ["MambaForCausalLM"], "model_type": "mamba"})
    with pytest.raises(ConfigError):
        resolve_architecture({})
    (tmp_path / "config.json").write_text(json.dumps(TINY_W))
    arch, cfg = load_config(str(tmp_path))
    spec = arch.describe(cfg)
    assert len(spec.layers) == 3 and spec.layers[0].mixer.params["window"] == 40
    assert spec.layers[1].mixer.params["window"] is None
    (tmp_path / "config.json").write_text("{ not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))


def test_another_architecture_can_be_registered():
    toy = Architecture("ToyForCausalLM", parse=Qwen3Config.from_dict, describe=describe_qwen3)
    register_architecture(toy, replace=True)
    assert resolve_architecture({"architectures": ["ToyForCausalLM"]}) is toy
    with pytest.raises(ValueError):
        register_architecture(Architecture("ToyForCausalLM", parse=dict, describe=dict))


def test_model_description_holds_no_constants_of_its_own():
    c = Qwen3Config.from_dict(TINY_B)
    spec = describe_qwen3(c)
    m = spec.layers[0].mixer.params
    assert (m["num_heads"], m["num_kv_heads"], m["head_dim"], m["qk_norm_eps"]) == (8, 1, 32, 1e-5)
    assert m["scale"] == pytest.approx(32 ** -0.5)
    assert spec.position_encodings["rope"].params["theta"] == 1e6
    assert spec.head.params["tied"] is False and [e.layer for e in spec.schedule] == [0, 1, 2]


def test_generation_defaults(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_A, eos_token_id=7)))
    g = GenerationDefaults.from_dir(str(tmp_path))
    assert g.eos_token_ids == (7,) and g.temperature is None
    (tmp_path / "generation_config.json").write_text(json.dumps(
        dict(eos_token_id=[5, 6], temperature=0.6, top_p=0.95, top_k=20)))
    g = GenerationDefaults.from_dir(str(tmp_path))
    assert g.eos_token_ids == (5, 6) and g.temperature == pytest.approx(0.6) and g.top_k == 20


def test_a_head_size_no_kernel_takes_is_refused_when_the_model_is_described():
    """head_dim 24 is a valid config; the attention part says at once that its kernels take multiples
    of 16 only (the model is never built with a size that would first fail in a step)."""
    import torch
    from paged_llm_rs_b200 import KernelError
    from paged_llm_rs_b200.models.qwen3 import describe_qwen3
    from paged_llm_rs_b200.parts.base import Runtime
    from paged_llm_rs_b200.parts.decoder import DecoderModel

    d = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu", hidden_size=48, intermediate_size=64,
             num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1, head_dim=24, rms_norm_eps=1e-6,
             vocab_size=50, max_position_embeddings=64, tie_word_embeddings=True, rope_theta=10000.0)
    spec = describe_qwen3(Qwen3Config.from_dict(d))
    with pytest.raises(KernelError, match="head_dim 24"):
        DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32))
