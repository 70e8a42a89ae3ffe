"""Qwen3 dense decoder, described as parts.

Tensor names and shapes follow the checkpoint
(crates/pagedllm/src/model/mod.rs:174-236): per layer seven bias-free
projections stored [out, in] and four norm gains; q_norm / k_norm are as wide as
one head (mod.rs:199-203); the head prefers a stored ``lm_head.weight`` and
falls back to the embedding when the config ties them (mod.rs:222-235).
"""

from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.schema import Qwen3Config
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def describe_qwen3(cfg: Qwen3Config) -> ModelSpec:
    rope = PartSpec(
        "rope",
        dict(head_dim=cfg.head_dim, rotary_dim=cfg.head_dim, theta=cfg.rope_theta,
             max_positions=cfg.max_position_embeddings),
    )
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        norm = lambda name, width: PartSpec("rmsnorm", dict(width=width, eps=cfg.rms_norm_eps), f"{p}.{name}")
        layers.append(
            LayerSpec(
                block="prenorm_residual",
                mixer=PartSpec(
                    "gqa_attention",
                    dict(
                        hidden_size=cfg.hidden_size,
                        num_heads=cfg.num_attention_heads,
                        num_kv_heads=cfg.num_key_value_heads,
                        head_dim=cfg.head_dim,
                        qk_norm_eps=cfg.rms_norm_eps,  # per-head q/k RMSNorm (attention.rs:148-149)
                        scale=cfg.head_dim ** -0.5,  # attention.rs:51
                        window=cfg.window_of_layer(i),
                        position_encoding="rope",
                    ),
                    f"{p}.self_attn",
                ),
                feed_forward=PartSpec(
                    "swiglu_mlp",
                    dict(hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size),
                    f"{p}.mlp",
                ),
                norms={
                    "mixer": norm("input_layernorm", cfg.hidden_size),
                    "feed_forward": norm("post_attention_layernorm", cfg.hidden_size),
                },
                prefix=p,
            )
        )
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size),
                           "model.embed_tokens"),
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps), "model.norm"),
        head=PartSpec(
            "linear_head",
            dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, tied=cfg.tie_word_embeddings,
                 tied_to="model.embed_tokens.weight"),
            "lm_head",
        ),
        position_encodings={"rope": rope},
    )


QWEN3 = Architecture(
    name="Qwen3ForCausalLM",
    parse=Qwen3Config.from_dict,
    describe=describe_qwen3,
    aliases=("qwen3",),
)
register_architecture(QWEN3)
