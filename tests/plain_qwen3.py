"""A plain, slow Qwen3 for tests: whole sequences, no cache, one function per part.

It rests on the reference's formulas (nicoNaeg/paged-llm-rs), each function citing
the file and lines it restates.  The reference's own model code is Rust on candle
and cannot be compiled here (no cargo), so the anchor is its committed fixture:
``tests/golden/reference_fixture`` holds the tiny model and the 36 activations the
reference's tests compare with (crates/pagedllm/tests/forward.rs:23-51), and
``tests/test_plain.py`` checks this file against them.

It shares no code with the engine: weights are read with the ``safetensors``
library, not the engine's reader, and nothing is imported from the package.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch


def load_model(model_dir: str, dtype=torch.float32, device="cpu"):
    """config.json as a dict and every tensor of model.safetensors cast to ``dtype``
    (on ``device``: the functions below run wherever the weights are)."""
    from safetensors.torch import load_file

    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = {k: v.to(device=device, dtype=dtype) for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, w


def rope_theta(cfg) -> float:
    """Flat, or nested under rope_parameters (crates/pagedllm/src/config.rs:139-145)."""
    if cfg.get("rope_theta") is not None:
        return float(cfg["rope_theta"])
    return float(cfg["rope_parameters"]["rope_theta"])


def layer_window(cfg, layer: int) -> Optional[int]:
    """The window of a layer, or None.  The reference refuses windows
    (config.rs:104-106); this follows the config's own keys: a layer slides when
    use_sliding_window is set and layer_types (or max_window_layers) says so."""
    if not cfg.get("use_sliding_window"):
        return None
    types = cfg.get("layer_types")
    if types is None:
        first = cfg.get("max_window_layers", cfg["num_hidden_layers"])
        types = ["sliding_attention" if i >= first else "full_attention" for i in range(cfg["num_hidden_layers"])]
    return int(cfg["sliding_window"]) if types[layer] == "sliding_attention" else None


def embed(tokens: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x[t] = table[token[t]], no scaling (crates/pagedllm/src/model/mod.rs:282-283)."""
    return table[tokens]


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * gain over the last dimension, eps inside the root
    (crates/pagedllm/src/model/layers.rs:58-64)."""
    variance = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(variance + eps) * gain


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """y = x W^T, weight stored [out, in], no bias (layers.rs:19-35)."""
    return x @ weight.t()


def rope_tables(head_dim: int, positions: int, theta: float, dtype=torch.float32, device="cpu"):
    """cos/sin [positions, head_dim]: inv_freq[i] = 1/theta^(2i/head_dim), the angle
    pos*inv_freq[i] in float64, each angle twice (once per half of the head)
    (crates/pagedllm/src/model/rope.rs:39-62)."""
    half = head_dim // 2
    inv_freq = torch.tensor([1.0 / theta ** (2.0 * i / head_dim) for i in range(half)], dtype=torch.float64)
    angle = torch.arange(positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
    angle = torch.cat([angle, angle], dim=-1)
    return (angle.cos().to(torch.float32).to(device=device, dtype=dtype),
            angle.sin().to(torch.float32).to(device=device, dtype=dtype))


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """[x1, x2] -> [-x2, x1] over the last dimension (rope.rs:102-107)."""
    half = x.shape[-1] // 2
    return torch.cat([-x[..., half:], x[..., :half]], dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x*cos + rotate_half(x)*sin; x is [heads, seq, head_dim], tables [seq, head_dim]
    (rope.rs:96-99)."""
    return x * cos + rotate_half(x) * sin


def causal_mask(seq: int, window: Optional[int], dtype, device="cpu") -> torch.Tensor:
    """0 where key j <= query i, -inf past it (crates/pagedllm/src/model/attention.rs:255-275).
    With a window w, key j is also hidden when j <= i - w: a query sees itself and
    the w-1 keys before it (not in the reference, which has no window)."""
    i = torch.arange(seq, device=device)[:, None]
    j = torch.arange(seq, device=device)[None, :]
    hidden = j > i
    if window is not None:
        hidden = hidden | (j <= i - window)
    return torch.zeros(seq, seq, dtype=dtype, device=device).masked_fill(hidden, float("-inf"))


def softmax_last(x: torch.Tensor) -> torch.Tensor:
    """exp(x - max) / sum (attention.rs:282-289)."""
    e = torch.exp(x - x.max(dim=-1, keepdim=True).values)
    return e / e.sum(dim=-1, keepdim=True)


def attention(x, w: Dict[str, torch.Tensor], prefix: str, cfg, cos, sin, window, trace=None):
    """q/k/v projections, split into heads, per-head RMSNorm of q and k, RoPE, grouped
    heads (query head h reads key head h // group), scaled scores, causal mask,
    softmax, weighted sum, output projection (attention.rs:62-114, 240-248)."""
    seq = x.shape[0]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    q = linear(x, w[f"{prefix}.q_proj.weight"])
    k = linear(x, w[f"{prefix}.k_proj.weight"])
    v = linear(x, w[f"{prefix}.v_proj.weight"])
    if trace is not None:
        trace[f"{prefix}.q_proj.out"], trace[f"{prefix}.k_proj.out"], trace[f"{prefix}.v_proj.out"] = q, k, v
    q = rms_norm(q.reshape(seq, nh, hd), w[f"{prefix}.q_norm.weight"], eps)
    k = rms_norm(k.reshape(seq, nkv, hd), w[f"{prefix}.k_norm.weight"], eps)
    v = v.reshape(seq, nkv, hd)
    if trace is not None:
        trace[f"{prefix}.q_norm.out"], trace[f"{prefix}.k_norm.out"] = q, k
    q = apply_rope(q.transpose(0, 1), cos[:seq], sin[:seq])  # [nh, seq, hd]
    k = apply_rope(k.transpose(0, 1), cos[:seq], sin[:seq])
    v = v.transpose(0, 1)
    group = nh // nkv
    k = k.repeat_interleave(group, dim=0)  # head h reads kv head h // group
    v = v.repeat_interleave(group, dim=0)
    scores = q @ k.transpose(-1, -2) * (1.0 / math.sqrt(hd))
    scores = scores + causal_mask(seq, window, scores.dtype, scores.device)
    out = softmax_last(scores) @ v  # [nh, seq, hd]
    out = out.transpose(0, 1).reshape(seq, nh * hd)
    if trace is not None:
        trace[f"{prefix}.o_proj.in"] = out
    out = linear(out, w[f"{prefix}.o_proj.weight"])
    if trace is not None:
        trace[f"{prefix}.o_proj.out"] = out
        trace[f"{prefix}.out"] = out
    return out


def swiglu_mlp(x, w, prefix: str, trace=None):
    """down(silu(gate(x)) * up(x)); the gate carries the activation (layers.rs:93-105)."""
    gate = linear(x, w[f"{prefix}.gate_proj.weight"])
    up = linear(x, w[f"{prefix}.up_proj.weight"])
    gated = gate * torch.sigmoid(gate) * up
    out = linear(gated, w[f"{prefix}.down_proj.weight"])
    if trace is not None:
        trace[f"{prefix}.gate_proj.out"], trace[f"{prefix}.up_proj.out"] = gate, up
        trace[f"{prefix}.down_proj.in"], trace[f"{prefix}.down_proj.out"] = gated, out
        trace[f"{prefix}.out"] = out
    return out


def block(x, w, layer: int, cfg, cos, sin, trace=None):
    """x + attn(norm(x)), then x + mlp(norm(x)) (model/mod.rs:92-114)."""
    p = f"model.layers.{layer}"
    eps = cfg["rms_norm_eps"]
    normed = rms_norm(x, w[f"{p}.input_layernorm.weight"], eps)
    if trace is not None:
        trace[f"{p}.input_layernorm.out"] = normed
    x = x + attention(normed, w, f"{p}.self_attn", cfg, cos, sin, layer_window(cfg, layer), trace)
    normed = rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], eps)
    if trace is not None:
        trace[f"{p}.post_attention_layernorm.out"] = normed
    x = x + swiglu_mlp(normed, w, f"{p}.mlp", trace)
    if trace is not None:
        trace[f"{p}.out"] = x
    return x


def forward(cfg, w, tokens: List[int], trace: Optional[dict] = None, rows: Optional[List[int]] = None) -> torch.Tensor:
    """Logits [len(tokens), vocab] of one sequence from position 0, every position
    projected (model/mod.rs:271-303); with ``rows``, only those positions are normed
    and projected (mod.rs:340-351).  The head is lm_head.weight when stored, else
    the embedding when tied, else an error (mod.rs:226-235)."""
    if not tokens:
        raise ValueError("cannot run a forward pass on no tokens")
    dtype, device = w["model.embed_tokens.weight"].dtype, w["model.embed_tokens.weight"].device
    ids = torch.tensor(tokens, dtype=torch.long, device=device)
    x = embed(ids, w["model.embed_tokens.weight"])
    if trace is not None:
        trace["model.embed_tokens.out"] = x
    cos, sin = rope_tables(cfg["head_dim"], len(tokens), rope_theta(cfg), dtype, device)
    for layer in range(cfg["num_hidden_layers"]):
        x = block(x, w, layer, cfg, cos, sin, trace)
    if rows is not None:
        x = x[torch.tensor(list(rows), dtype=torch.long, device=device)]
    x = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    if "lm_head.weight" in w:
        head = w["lm_head.weight"]
    elif cfg["tie_word_embeddings"]:
        head = w["model.embed_tokens.weight"]
    else:
        raise ValueError("no lm_head.weight, and the config does not tie the embeddings")
    logits = linear(x, head)
    if trace is not None:
        trace["model.norm.out"] = x
        trace["lm_head.out"] = logits
        trace["logits"] = logits
    return logits


# --- sampling (crates/pagedllm/src/sampler.rs) --------------------------------

MASK64 = (1 << 64) - 1


class PlainRng:
    """splitmix64 (sampler.rs:23-43): state += 0x9E3779B97F4A7C15 per call."""

    def __init__(self, seed: int):
        self.state = seed & MASK64

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & MASK64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
        return z ^ (z >> 31)

    def next_f32(self) -> float:
        """Top 24 bits over 2^24: a number in [0, 1) (sampler.rs:41-43)."""
        return (self.next_u64() >> 40) / float(1 << 24)


def greedy(logits: torch.Tensor) -> int:
    """First maximum wins (sampler.rs:186-194)."""
    best = 0
    vals = logits.tolist()
    for i, v in enumerate(vals):
        if v > vals[best]:
            best = i
    return best


def sample(logits: torch.Tensor, temperature: float, top_k: Optional[int], top_p: Optional[float],
           rng: PlainRng) -> int:
    """temperature, top-k, softmax over the survivors in descending order, top-p
    keeping the token that crosses p, then walk the draw down the sorted weights
    (sampler.rs:113-183).  Equal logits are ordered by id, which the reference
    leaves open (sort_unstable, sampler.rs:144)."""
    import numpy as np

    if temperature <= 0.0:
        return greedy(logits)
    inv = np.float32(1.0) / np.float32(temperature)
    scaled = logits.to(torch.float32).numpy().astype(np.float32) * inv
    cand = sorted(range(len(scaled)), key=lambda i: (-float(scaled[i]), i))
    if top_k is not None and top_k < len(cand):
        cand = cand[:top_k]
    largest = scaled[cand[0]]
    weights = [np.exp(np.float32(scaled[i] - largest), dtype=np.float32) for i in cand]
    total = np.float32(0.0)
    for x in weights:
        total = np.float32(total + x)
    if top_p is not None and top_p < 1.0:
        target = np.float32(top_p) * total
        running = np.float32(0.0)
        keep = 1
        for pos, x in enumerate(weights):
            running = np.float32(running + x)
            keep = pos + 1
            if running >= target:
                break
        cand, weights = cand[:keep], weights[:keep]
        total = np.float32(0.0)
        for x in weights:
            total = np.float32(total + x)
    point = np.float32(rng.next_f32()) * total
    for i, x in zip(cand, weights):
        point = np.float32(point - x)
        if point <= 0.0:
            return i
    return cand[-1]
