"""Toy parts of every kind, defined and registered here, built into one model and stepped through
the engine's own runner, cache and captured steps without a change to the framework's files:

  a feed-forward with routing (a router in float32, the best two of five small gated experts),
  another position encoding (a learned row for every absolute position, added behind the embedding,
  with an attention layer that does not rotate),
  another norm (mean and variance, gain and bias),
  another arrangement of a block (mixer and feed-forward side by side on one norm).

They are toys for the interfaces: plain tensor code on the device, no model of anyone's.  The plain
implementation of the whole toy model stands below, in float64 over whole sequences.
"""

import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from paged_llm_rs_b200.config import Architecture, Qwen3Config, register_architecture
from paged_llm_rs_b200.engine.runner import ModelRunner
from paged_llm_rs_b200.engine.step import StepEntry
from paged_llm_rs_b200.models.qwen3 import describe_qwen3
from paged_llm_rs_b200.parts.base import (Block, FeedForward, Norm, PositionEncoding, register_block,
                                          register_feed_forward, register_norm, register_position_encoding)
from paged_llm_rs_b200.parts.spec import ModelSpec, PartSpec, TensorSpec
from paged_llm_rs_b200.weights.random_init import write_random_model
from tiny_configs import TINY_C

EXPERTS, TOP_K, EXPERT_SIZE, LN_EPS = 5, 2, 24, 1e-5


class RoutedFeedForward(FeedForward):
    """Router logits and their softmax in float32; the best ``top_k`` experts of a token, their
    weights made to sum to one; every expert a small gated feed-forward.  Every expert runs on every
    token and the unchosen ones are weighted zero, so that the launches do not depend on the routing
    (a captured step replays them)."""

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = spec.params
        self.hidden, self.experts, self.top_k, self.size = p["hidden_size"], p["experts"], p["top_k"], p["expert_size"]

    def tensors(self):
        t = [TensorSpec(self._name("router.weight"), (self.experts, self.hidden))]
        for e in range(self.experts):
            t += [TensorSpec(self._name(f"experts.{e}.gate.weight"), (self.size, self.hidden)),
                  TensorSpec(self._name(f"experts.{e}.up.weight"), (self.size, self.hidden)),
                  TensorSpec(self._name(f"experts.{e}.down.weight"), (self.hidden, self.size))]
        return t

    def bind(self, tensors):
        self.router = tensors[self._name("router.weight")].float()
        self.gate = torch.stack([tensors[self._name(f"experts.{e}.gate.weight")] for e in range(self.experts)])
        self.up = torch.stack([tensors[self._name(f"experts.{e}.up.weight")] for e in range(self.experts)])
        self.down = torch.stack([tensors[self._name(f"experts.{e}.down.weight")] for e in range(self.experts)])

    def forward(self, x, step):
        prob = torch.softmax(x.float() @ self.router.t(), -1)
        best, which = prob.topk(self.top_k, -1)
        share = torch.zeros_like(prob).scatter_(1, which, best / best.sum(-1, keepdim=True))     # [tokens, experts]
        g = torch.einsum("th,esh->ets", x, self.gate)
        u = torch.einsum("th,esh->ets", x, self.up)
        act = (torch.nn.functional.silu(g.float()) * u.float()).to(x.dtype)
        y = torch.einsum("ets,ehs->eth", act, self.down).float()
        return (y * share.t()[:, :, None]).sum(0).to(x.dtype)


class LearnedPositions(PositionEncoding):
    """A learned row for every absolute position, added to the residual stream behind the embedding."""

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden, self.max_positions = spec.params["hidden_size"], spec.params["max_positions"]

    def tensors(self):
        return [TensorSpec(self._name("weight"), (self.max_positions, self.hidden))]

    def bind(self, tensors):
        self.table = tensors[self._name("weight")]

    def at_embedding(self, hidden, step):
        return hidden + self.table.index_select(0, step.positions[:hidden.shape[0]].long())


class MeanVarianceNorm(Norm):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.width, self.eps = spec.params["width"], spec.params["eps"]

    def tensors(self):
        return [TensorSpec(self._name("weight"), (self.width,), "gain"), TensorSpec(self._name("bias"), (self.width,))]

    def bind(self, tensors):
        self.gain, self.bias = tensors[self._name("weight")].float(), tensors[self._name("bias")].float()

    def forward(self, x, rows=None):
        if rows is not None:
            x = x.index_select(0, rows.long())
        f = x.float()
        f = f - f.mean(-1, keepdim=True)
        return (f * torch.rsqrt(f.square().mean(-1, keepdim=True) + self.eps) * self.gain + self.bias).to(x.dtype)


class SideBySideBlock(Block):
    """x + mixer(norm(x)) + feed_forward(norm(x)): one norm, both parts read it."""

    def forward(self, residual, delta, step, cache, writes_cache=True):
        h = self.norms["shared"].add_norm(residual, delta)
        return residual, self.mixer.forward(h, step, cache, writes_cache) + self.feed_forward.forward(h, step)


def describe_toy_parts(cfg: Qwen3Config) -> ModelSpec:
    spec = describe_qwen3(cfg)
    H = cfg.hidden_size
    spec.position_encodings["learned"] = PartSpec("toy_learned_positions",
                                                  dict(hidden_size=H, max_positions=cfg.max_position_embeddings),
                                                  "model.positions")
    first, second = spec.layers
    # layer 0: attention that does not rotate (the learned rows place the tokens), beside its
    # feed-forward on one norm of the other kind
    first.block = "toy_side_by_side"
    first.mixer.params["position_encoding"] = None
    first.norms = {"shared": PartSpec("toy_mean_variance_norm", dict(width=H, eps=LN_EPS), "model.layers.0.ln")}
    # layer 1: Qwen3's own block and rotating attention, with the routed feed-forward
    second.feed_forward = PartSpec("toy_routed", dict(hidden_size=H, experts=EXPERTS, top_k=TOP_K, expert_size=EXPERT_SIZE),
                                   "model.layers.1.moe")
    return spec


def register_toys():
    register_feed_forward("toy_routed", RoutedFeedForward, replace=True)
    register_position_encoding("toy_learned_positions", LearnedPositions, replace=True)
    register_norm("toy_mean_variance_norm", MeanVarianceNorm, replace=True)
    register_block("toy_side_by_side", SideBySideBlock, replace=True)
    register_architecture(Architecture("ToyPartsForCausalLM", parse=lambda d: Qwen3Config.from_dict(dict(d, model_type="qwen3")),
                                       describe=describe_toy_parts), replace=True)


TOY = dict(TINY_C, architectures=["ToyPartsForCausalLM"], model_type="toy_parts")


def plain_toy_parts(model_dir, tokens):
    """(logits [n, vocab], per token the distance between the router's second and third logit)."""
    cfg, w = P.load_model(model_dir, torch.float64)
    n = len(tokens)
    eps = cfg["rms_norm_eps"]
    cos, sin = P.rope_tables(cfg["head_dim"], n, cfg["rope_theta"], torch.float64)
    x = P.embed(torch.tensor(tokens), w["model.embed_tokens.weight"]) + w["model.positions.weight"][:n]

    # layer 0
    f = x - x.mean(-1, keepdim=True)
    h = f / torch.sqrt(f.square().mean(-1, keepdim=True) + LN_EPS) * w["model.layers.0.ln.weight"] + w["model.layers.0.ln.bias"]
    no_turn = (torch.ones_like(cos), torch.zeros_like(sin))
    x = x + P.attention(h, w, "model.layers.0.self_attn", cfg, *no_turn, None) + P.swiglu_mlp(h, w, "model.layers.0.mlp")

    # layer 1
    p = "model.layers.1"
    x = x + P.attention(P.rms_norm(x, w[f"{p}.input_layernorm.weight"], eps), w, f"{p}.self_attn", cfg, cos, sin, None)
    h = P.rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], eps)
    logit = h @ w[f"{p}.moe.router.weight"].t()
    prob = P.softmax_last(logit)
    out = torch.zeros_like(h)
    for t in range(n):
        order = sorted(range(EXPERTS), key=lambda e: -float(prob[t, e]))[:TOP_K]
        total = sum(prob[t, e] for e in order)
        for e in order:
            q = f"{p}.moe.experts.{e}"
            g, u = w[f"{q}.gate.weight"] @ h[t], w[f"{q}.up.weight"] @ h[t]
            out[t] += prob[t, e] / total * (w[f"{q}.down.weight"] @ (g / (1 + torch.exp(-g)) * u))
    x = x + out
    ranked = logit.sort(-1, descending=True).values
    margin = (ranked[:, TOP_K - 1] - ranked[:, TOP_K]) / ranked.abs().max(-1).values
    logits = P.linear(P.rms_norm(x, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])
    return logits.numpy(), margin.numpy()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_feed_forward_position_encoding_norm_and_block(tmp_path, dtype):
    register_toys()
    model = write_random_model(str(tmp_path / "toy_parts"), TOY, 11, matrix_std=0.05)
    runner = ModelRunner(model, dtype=dtype, page_size=8, num_pages=16, max_requests=4)
    assert runner.use_graphs
    cache = runner.cache
    rng = np.random.default_rng(4)
    steps = 5
    lens = dict(a=30, b=21, c=9)
    toks = {r: rng.integers(0, 1000, n + steps).tolist() for r, n in lens.items()}
    got, fed = {r: {} for r in toks}, {r: 0 for r in toks}

    def run(parts):
        entries = []
        for r, n in parts:
            if not cache.has(r):
                cache.open(r)
            assert cache.reserve(r, n)
            entries.append(StepEntry(r, toks[r][fed[r]:fed[r] + n], list(range(n))))
        logits = runner.step(entries).cpu().numpy()
        row = 0
        for e in entries:
            for i in range(len(e.tokens)):
                got[e.request_id][fed[e.request_id] + i] = logits[row]; row += 1
            cache.commit(e.request_id, len(e.tokens))
            fed[e.request_id] += len(e.tokens)

    # portions beside single tokens, down to two tokens
    run([("a", 11)]); run([("a", 2), ("b", 9)]); run([("a", 1), ("b", 1)]); run([("b", 11), ("a", 16)]); run([("c", 9)])
    # then the three decode through the captured step (made for four: one row of padding)
    zeros = np.zeros(3, dtype=np.float32)
    for i in range(steps):
        entries = [StepEntry(r, [toks[r][lens[r] + i]], [0]) for r in lens]
        for r in lens:
            assert cache.reserve(r, 1)
        logits, tokens = runner.step_and_sample(entries, zeros, zeros)
        logits = logits.cpu().numpy()
        assert runner._decode_graph(entries).graph is not None          # one captured piece: every toy is capturable
        assert (tokens.cpu().numpy()[1:] == logits.argmax(1)).all()
        for row, r in enumerate(lens):
            got[r][lens[r] + i] = logits[row]
            cache.commit(r, 1)
    runner.check_status()

    t = 2e-5 if dtype == "float32" else 3e-2
    compared = total = 0
    for r in toks:
        want, margin = plain_toy_parts(model, toks[r])
        # A token whose second and third expert lie closer than bfloat16 resolves may be routed the
        # other way; the choice is a step in the function, so such tokens are left out in bfloat16
        # (the routed layer is the last one: its output reaches no other token).
        clear = margin > (0.0 if dtype == "float32" else 0.05)
        total += len(clear)
        compared += int(clear.sum())
        have = np.stack([got[r][i] for i in range(len(toks[r]))])
        err = np.abs(have - want).max(-1) / max(1.0, np.abs(want).max())
        assert (err[clear] <= t).all(), (r, np.nonzero(clear & (err > t))[0], err.max())
    assert compared >= 0.8 * total
    for r in lens:
        cache.close(r)
    cache.check_invariants()
    assert cache.available() == 16


def test_the_toy_parts_matter():
    """The plain toy model with a part taken out gives other logits: the comparison above would see a
    framework that skipped the learned rows, the routing or the bias."""
    import tempfile
    register_toys()
    with tempfile.TemporaryDirectory() as d:
        model = write_random_model(d + "/toy_parts", TOY, 11, matrix_std=0.05)
        tokens = np.random.default_rng(0).integers(0, 1000, 24).tolist()
        want, _ = plain_toy_parts(model, tokens)
        from safetensors.torch import load_file, save_file
        stored = load_file(model + "/model.safetensors")
        for name in ("model.positions.weight", "model.layers.1.moe.router.weight", "model.layers.0.ln.bias"):
            changed = dict(stored)
            changed[name] = torch.zeros_like(stored[name])
            save_file(changed, model + "/model.safetensors")
            other, _ = plain_toy_parts(model, tokens)
            assert np.abs(other - want).max() / max(1.0, np.abs(want).max()) > 1e-3, name
