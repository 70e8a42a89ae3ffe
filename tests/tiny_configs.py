"""Two tiny Qwen3 configurations that differ in every size and option, and
helpers that write them as model folders with random weights."""

import os

TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu", attention_bias=False,
    hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
    head_dim=16, rms_norm_eps=1e-6, vocab_size=256, max_position_embeddings=512, tie_word_embeddings=True,
    rope_theta=10000.0, sliding_window=None, use_sliding_window=False,
)

# heads * head_dim != hidden, one kv head (8 query heads share it), sizes that are no
# power of two, untied head, nested rope_theta, another eps; every layer keeps every key,
# so equal prefixes are shared.  Served on pages of 8.
TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
    hidden_size=96, intermediate_size=160, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=1,
    head_dim=32, rms_norm_eps=1e-5, vocab_size=384, max_position_embeddings=640, tie_word_embeddings=False,
    rope_parameters=dict(rope_theta=1000000.0, rope_type="default"),
)

# the same sizes with a window of 40 keys on two of the three layers (an extra: the reference
# refuses windows, so nothing of the reference pins this one but the config's own keys)
TINY_W = dict(TINY_B, use_sliding_window=True, sliding_window=40,
              layer_types=["sliding_attention", "full_attention", "sliding_attention"])

# a third one for kernels' odd sizes: head_dim 48, 6 heads over 3 kv heads, vocabulary 1000
TINY_C = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
    hidden_size=72, intermediate_size=200, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=3,
    head_dim=48, rms_norm_eps=1e-6, vocab_size=1000, max_position_embeddings=512, tie_word_embeddings=True,
    rope_theta=50000.0,
)

# a fourth one at the sizes the tensor-core kernels take: head_dim 64, widths that are
# multiples of 128, a window on its middle layer
TINY_D = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
    hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
    head_dim=64, rms_norm_eps=1e-6, vocab_size=512, max_position_embeddings=1024, tie_word_embeddings=True,
    rope_theta=1000000.0, use_sliding_window=True, sliding_window=70,
    layer_types=["full_attention", "sliding_attention", "full_attention"],
)

CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3), "W": (TINY_W, 4)}
PAGE_SIZES = {"A": 16, "B": 8, "C": 16, "D": 16, "W": 16}

# Matrices drawn from N(0, 0.02) give a tied model that mostly repeats its last token: its
# greedy tokens say little about attention or the cache.  Folders for checks on TOKENS are
# therefore drawn five times wider and with a head of their own: there the plain
# implementation's argmax changes at (nearly) every position when the attention output is
# zeroed (tests/test_plain.py checks it).  Checks on LOGITS keep N(0, 0.02).
DECISIVE_STD = 0.1


def write_model(folder, name, dtype=None, decisive=False):
    import torch
    from paged_llm_rs_b200.weights.random_init import write_random_model

    cfg, seed = CONFIGS[name]
    d = os.path.join(str(folder), f"tiny_{name}" + ("_decisive" if decisive else ""))
    if decisive:
        write_random_model(d, dict(cfg, tie_word_embeddings=False), seed, dtype or torch.bfloat16,
                           matrix_std=DECISIVE_STD)
    else:
        write_random_model(d, cfg, seed, dtype or torch.bfloat16)
    return d
