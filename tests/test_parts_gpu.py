"""Each part alone against the plain implementation's function for it, and the
openness of the assembly: a toy mixer with state of its own, a schedule that
runs a layer twice and lets a run read another run's cache, all defined here and
registered, built and stepped without a change to the framework's files."""

import json
import math
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from paged_llm_rs_b200.cache import CacheManager
from paged_llm_rs_b200.config import Architecture, Qwen3Config, register_architecture
from paged_llm_rs_b200.engine.runner import ModelRunner
from paged_llm_rs_b200.engine.step import GroupPlanConfig, StepEntry, StepPacker
from paged_llm_rs_b200.kernels import ops
from paged_llm_rs_b200.models.qwen3 import describe_qwen3
from paged_llm_rs_b200.parts import base
from paged_llm_rs_b200.parts.base import Mixer, Runtime, StateNeed, register_mixer
from paged_llm_rs_b200.parts.decoder import DecoderModel
from paged_llm_rs_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec
from paged_llm_rs_b200.weights.random_init import write_random_model
from tiny_configs import TINY_B, TINY_C

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)


def rand(shape, seed, std=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * std


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    rt = Runtime(DEV, dtype)
    n = base.make(base.NORMS, "norm", PartSpec("rmsnorm", dict(width=72, eps=1e-5), "n"), rt)
    assert n.tensors() == [TensorSpec("n.weight", (72,), "gain")]
    gain = 1 + rand(72, 0, 0.1)
    n.bind({"n.weight": gain.to(DEV)})
    x, d = rand((5, 72), 1).to(dtype), rand((5, 72), 2).to(dtype)
    torch.testing.assert_close(n.forward(x.to(DEV)).float().cpu(), P.rms_norm(x.float(), gain, 1e-5), **tol(dtype))
    res = x.to(DEV).clone()
    y = n.add_norm(res, d.to(DEV))
    s = (x.float() + d.float()).to(dtype)
    assert torch.equal(res.cpu(), s)
    torch.testing.assert_close(y.float().cpu(), P.rms_norm(s.float(), gain, 1e-5), **tol(dtype))


def test_rotary_tables_match_the_plain_ones():
    rt = Runtime(DEV, torch.float32)
    enc = base.make(base.POSITION_ENCODINGS, "position encoding",
                    PartSpec("rope", dict(head_dim=48, theta=1e6, max_positions=300)), rt)
    cos, sin, rdim = enc.rotary()
    pc, psn = P.rope_tables(48, 300, 1e6)
    assert rdim == 48 and torch.equal(cos.cpu(), pc[:, :24]) and torch.equal(sin.cpu(), psn[:, :24])


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_embedding_and_head_parts(dtype):
    rt = Runtime(DEV, dtype)
    ff = base.make(base.FEED_FORWARDS, "feed-forward", PartSpec("swiglu_mlp", dict(hidden_size=72, intermediate_size=200), "m"), rt)
    w = {"m.gate_proj.weight": rand((200, 72), 1, 0.1).to(dtype), "m.up_proj.weight": rand((200, 72), 2, 0.1).to(dtype),
         "m.down_proj.weight": rand((72, 200), 3, 0.1).to(dtype)}
    assert sorted(t.name for t in ff.tensors()) == sorted(w)
    ff.bind({k: v.to(DEV) for k, v in w.items()})
    x = rand((9, 72), 4).to(dtype)
    want = P.swiglu_mlp(x.float(), {k: v.float() for k, v in w.items()}, "m")
    torch.testing.assert_close(ff.forward(x.to(DEV), None).float().cpu(), want, **tol(dtype))

    emb = base.make(base.EMBEDDINGS, "embedding", PartSpec("token_embedding", dict(vocab_size=1000, hidden_size=72), "e"), rt)
    table = rand((1000, 72), 5).to(dtype)
    table_dev = table.to(DEV)
    emb.bind({"e.weight": table_dev})
    toks = torch.tensor([0, 999, 17], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(toks).cpu(), table[[0, 999, 17]])

    # the head: its own tensor when the file has one, else the embedding when tied, else an error
    from paged_llm_rs_b200.errors import WeightError
    spec = PartSpec("linear_head", dict(vocab_size=1000, hidden_size=72, tied=True, tied_to="e.weight"), "h")
    head = base.make(base.HEADS, "head", spec, rt)
    head.bind({"e.weight": table_dev})
    logits = head.forward(x.to(DEV))
    assert logits.dtype == torch.float32 and head.weight.data_ptr() == emb.table.data_ptr()   # no copy when tied
    torch.testing.assert_close(logits.cpu(), x.float() @ table.float().T, **tol(dtype))
    own = rand((1000, 72), 6).to(dtype)
    head.bind({"e.weight": table_dev, "h.weight": own.to(DEV)})
    torch.testing.assert_close(head.forward(x.to(DEV)).cpu(), x.float() @ own.float().T, **tol(dtype))
    untied = base.make(base.HEADS, "head", PartSpec("linear_head", dict(vocab_size=1000, hidden_size=72, tied=False), "h"), rt)
    with pytest.raises(WeightError, match="does not tie"):
        untied.bind({})


def attention_weights(cfg, prefix, seed):
    nh, nkv, hd, H = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["hidden_size"]
    return {f"{prefix}.q_proj.weight": rand((nh * hd, H), seed, 0.15), f"{prefix}.k_proj.weight": rand((nkv * hd, H), seed + 1, 0.15),
            f"{prefix}.v_proj.weight": rand((nkv * hd, H), seed + 2, 0.15), f"{prefix}.o_proj.weight": rand((H, nh * hd), seed + 3, 0.15),
            f"{prefix}.q_norm.weight": 1 + rand(hd, seed + 4, 0.1), f"{prefix}.k_norm.weight": 1 + rand(hd, seed + 5, 0.1)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_alone_in_portions(dtype, window):
    """The mixer alone: 40 tokens in portions of 13, 2, 24 and a decoded one, through
    pages of 8, against the plain attention over the whole sequence."""
    cfg = dict(TINY_C)
    rt = Runtime(DEV, dtype)
    nh, nkv, hd, H = 6, 3, 48, 72
    enc = base.make(base.POSITION_ENCODINGS, "position encoding",
                    PartSpec("rope", dict(head_dim=hd, theta=50000.0, max_positions=64)), rt)
    att = base.make(base.MIXERS, "mixer", PartSpec("gqa_attention", dict(
        hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd, qk_norm_eps=1e-6, scale=hd ** -0.5,
        window=window, position_encoding="rope"), "a"), rt, position_encodings={"rope": enc})
    w = {k: v.to(dtype) if "norm" not in k else v for k, v in attention_weights(cfg, "a", 10).items()}
    att.bind({k: v.to(DEV) for k, v in w.items()})
    cache = CacheManager([att.cache_need()], 8, 12, 4, dtype, DEV, prefix_cache=False)
    wish = att.plan_wish(8)
    assert (wish.heads, wish.head_dim, wish.ctas_per_item) == (nh, hd, nkv)
    packer = StepPacker(cache, [GroupPlanConfig(wish.tile_tokens, wish.ctas_per_item, window, wish.heads, wish.head_dim)],
                        296, 1000, 64, DEV)
    x = rand((40, H), 20).to(dtype)
    cache.open("r")
    outs, p = [], 0
    for n in (13, 2, 24, 1):
        assert cache.reserve("r", n)
        host, layout, sizes = packer.pack([StepEntry("r", [0] * n, [])])
        state = packer.to_state(torch.from_numpy(host).to(DEV), layout, sizes)
        outs.append(att.forward(x[p:p + n].to(DEV).contiguous(), state, cache.layer_caches()[0]))
        cache.commit("r", n)
        p += n
    assert rt.status.item() == 0
    cos, sin = P.rope_tables(hd, 40, 50000.0)
    want = P.attention(x.float(), {k: v.float() for k, v in w.items()}, "a", cfg, cos, sin, window)
    torch.testing.assert_close(torch.cat(outs).float().cpu(), want, **tol(dtype))


# --- a toy mixer with state of its own, defined here -------------------------------------

class RunningMeanMixer(Mixer):
    """y_t = W * mean(x_0 .. x_t) over the tokens of the request so far.  Its state is
    fixed in size: the sum of the inputs and their count, kept in the request's slot."""

    def __init__(self, spec, rt, position_encodings=None):
        super().__init__(spec, rt)
        self.hidden = spec.params["hidden_size"]
        self.w = None

    def tensors(self):
        return [TensorSpec(self._name("mix.weight"), (self.hidden, self.hidden))]

    def bind(self, tensors):
        self.w = tensors[self._name("mix.weight")]

    def cache_need(self):
        return StateNeed((self.hidden + 1,), torch.float32)

    def forward(self, x, step, cache, writes_cache=True):
        out = torch.empty_like(x)
        for t0, n, before, slot in step.host_segments:
            s = cache[slot]
            sums = s[:-1] + torch.cumsum(x[t0:t0 + n].float(), 0)
            counts = s[-1] + torch.arange(1, n + 1, device=x.device)
            out[t0:t0 + n] = ((sums / counts[:, None]).to(x.dtype) @ self.w.t())
            if writes_cache:
                s[:-1] = sums[-1]
                s[-1] = counts[-1]
        return out


def describe_toy(cfg: Qwen3Config) -> ModelSpec:
    spec = describe_qwen3(cfg)
    # layer 0 keeps Qwen3's attention; layer 1 gets the toy mixer
    spec.layers[1].mixer = PartSpec("running_mean", dict(hidden_size=cfg.hidden_size), "model.layers.1.toy")
    # layer 0 runs twice; its second run reads the first run's cache; the toy layer runs twice, each run with state of its own
    spec.schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0, reads_cache_of=0), ScheduleEntry(1)]
    return spec


TOY = dict(TINY_C, architectures=["ToyStateForCausalLM"], model_type="toy_state")


def parse_toy(d):
    return Qwen3Config.from_dict(dict(d, model_type="qwen3"))


def plain_toy(model_dir, tokens):
    """The toy model's logits with the plain implementation's functions, whole sequence."""
    cfg, w = P.load_model(model_dir, torch.float64)
    n = len(tokens)
    x = P.embed(torch.tensor(tokens), w["model.embed_tokens.weight"])
    cos, sin = P.rope_tables(cfg["head_dim"], n, cfg["rope_theta"], torch.float64)
    eps = cfg["rms_norm_eps"]

    def toy(h):
        mean = torch.cumsum(h, 0) / torch.arange(1, n + 1, dtype=h.dtype)[:, None]
        return mean @ w["model.layers.1.toy.mix.weight"].t()

    def attn_reading_first_run(h, k_src):
        # queries from this run, keys and values from the first run's input
        p = "model.layers.0.self_attn"
        nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        q = P.rms_norm(P.linear(h, w[f"{p}.q_proj.weight"]).reshape(n, nh, hd), w[f"{p}.q_norm.weight"], eps)
        k = P.rms_norm(P.linear(k_src, w[f"{p}.k_proj.weight"]).reshape(n, nkv, hd), w[f"{p}.k_norm.weight"], eps)
        v = P.linear(k_src, w[f"{p}.v_proj.weight"]).reshape(n, nkv, hd)
        q, k = P.apply_rope(q.transpose(0, 1), cos, sin), P.apply_rope(k.transpose(0, 1), cos, sin)
        k, v = k.repeat_interleave(nh // nkv, 0), v.transpose(0, 1).repeat_interleave(nh // nkv, 0)
        s = q @ k.transpose(-1, -2) / math.sqrt(hd) + P.causal_mask(n, None, q.dtype)
        o = (P.softmax_last(s) @ v).transpose(0, 1).reshape(n, nh * hd)
        return P.linear(o, w[f"{p}.o_proj.weight"])

    def block(x, layer, mixer):
        p = f"model.layers.{layer}"
        x = x + mixer(P.rms_norm(x, w[f"{p}.input_layernorm.weight"], eps))
        return x + P.swiglu_mlp(P.rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], eps), w, f"{p}.mlp")

    first_in = {}

    def attn0(h):
        first_in["h"] = h
        return P.attention(h, w, "model.layers.0.self_attn", cfg, cos, sin, None)

    x = block(x, 0, attn0)
    x = block(x, 1, toy)
    x = block(x, 0, lambda h: attn_reading_first_run(h, first_in["h"]))
    x = block(x, 1, toy)
    x = P.rms_norm(x, w["model.norm.weight"], eps)
    return P.linear(x, w["model.embed_tokens.weight"]).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_and_schedule_without_touching_the_framework(tmp_path, dtype):
    register_mixer("running_mean", RunningMeanMixer, replace=True)
    register_architecture(Architecture("ToyStateForCausalLM", parse=parse_toy, describe=describe_toy), replace=True)
    model = write_random_model(str(tmp_path / "toy"), TOY, 3)
    runner = ModelRunner(model, dtype=dtype, page_size=8, num_pages=16, max_requests=4)
    cache = runner.cache
    assert len(cache.groups) == 1 and cache.groups[0].entries == [0]      # the second run of layer 0 owns no pages
    assert sorted(cache._state_entries) == [1, 3] and not cache.prefix_cache
    rng = np.random.default_rng(0)
    toks = {r: rng.integers(0, 1000, n).tolist() for r, n in (("a", 30), ("b", 21))}
    want = {r: plain_toy(model, t) for r, t in toks.items()}
    got = {r: {} for r in toks}
    fed = {r: 0 for r in toks}

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

    run([("a", 11)]); run([("a", 2), ("b", 9)]); run([("a", 1), ("b", 1)]); run([("b", 11), ("a", 16)])
    t = 2e-5 if dtype == "float32" else 3e-2
    for r in toks:
        g = np.stack([got[r][i] for i in range(len(toks[r]))])
        assert np.abs(g - want[r]).max() / max(1.0, np.abs(want[r]).max()) <= t, r
    cache.close("a"); cache.close("b")
    cache.check_invariants()


# --- a second toy mixer: one latent row per token, kept in pages of its own shape ---------------

class LatentMeanMixer(Mixer):
    """c_t = W_c x_t (``latent`` values) is cached for every token, in pages, as one row a token:
    not keys and values per head.  y_t = W_o mean(c_0 .. c_t).  It asks for no attention work
    items: the group's block tables and write slots are all it reads of the step."""

    def __init__(self, spec, rt, position_encodings=None):
        super().__init__(spec, rt)
        self.hidden, self.latent = spec.params["hidden_size"], spec.params["latent"]

    def tensors(self):
        return [TensorSpec(self._name("down.weight"), (self.latent, self.hidden)),
                TensorSpec(self._name("up.weight"), (self.hidden, self.latent))]

    def bind(self, tensors):
        self.w_c, self.w_o = tensors[self._name("down.weight")], tensors[self._name("up.weight")]

    def cache_need(self):
        return base.RowNeed(self.latent)

    def forward(self, x, step, cache, writes_cache=True):
        rows, gi = cache                                     # [pages, page_size, latent]
        g = step.groups[gi]
        assert g.plan is None
        c = x @ self.w_c.t()
        flat = rows.view(-1, self.latent)
        if writes_cache:
            slots = g.slots[:x.shape[0]].long()
            live = slots >= 0                                # (a captured step's padding has slot -1: nothing is written)
            flat[slots[live]] = c[live]
        out = torch.empty_like(x)
        ps = rows.shape[1]
        for si, (t0, n, before, slot) in enumerate(step.host_segments):
            total = before + n
            pages = g.block_tables[si, :-(-total // ps)].long()
            seen = rows[pages].reshape(-1, self.latent)[:total].float()
            mean = torch.cumsum(seen, 0)[before:] / torch.arange(before + 1, total + 1, device=x.device)[:, None]
            out[t0:t0 + n] = mean.to(x.dtype) @ self.w_o.t()
        return out


def describe_latent(cfg: Qwen3Config) -> ModelSpec:
    spec = describe_qwen3(cfg)
    spec.layers[1].mixer = PartSpec("latent_mean", dict(hidden_size=cfg.hidden_size, latent=40), "model.layers.1.latent")
    return spec


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_mixer_that_caches_one_latent_row_a_token_in_pages(tmp_path, dtype):
    register_mixer("latent_mean", LatentMeanMixer, replace=True)
    register_architecture(Architecture("ToyLatentForCausalLM", parse=parse_toy, describe=describe_latent), replace=True)
    cfg = dict(TINY_C, architectures=["ToyLatentForCausalLM"], model_type="toy_latent")
    model = write_random_model(str(tmp_path / "latent"), cfg, 5)
    runner = ModelRunner(model, dtype=dtype, page_size=8, num_pages=12, max_requests=4)
    cache = runner.cache
    # two groups with pages of different shapes: keys and values per head, and rows of 40 values
    assert [type(g.need).__name__ for g in cache.groups] == ["KVNeed", "RowNeed"]
    assert cache.groups[1].pool.shape == (1, 12, 8, 40) and runner.packer.plans[1] is None
    esz = 4 if dtype == "float32" else 2
    assert cache.bytes_per_token() == (2 * 3 * 48 + 40) * esz
    assert runner.use_graphs                                  # (captured around the toy, which loops over the step on the host)

    c64, w = P.load_model(model, torch.float64)

    def plain(tokens):
        n = len(tokens)
        x = P.embed(torch.tensor(tokens), w["model.embed_tokens.weight"])
        cos, sin = P.rope_tables(c64["head_dim"], n, c64["rope_theta"], torch.float64)
        eps = c64["rms_norm_eps"]

        def latent(h):
            c = h @ w["model.layers.1.latent.down.weight"].t()
            mean = torch.cumsum(c, 0) / torch.arange(1, n + 1, dtype=c.dtype)[:, None]
            return mean @ w["model.layers.1.latent.up.weight"].t()

        for layer, mixer in ((0, lambda h: P.attention(h, w, "model.layers.0.self_attn", c64, cos, sin, None)), (1, latent)):
            p = f"model.layers.{layer}"
            x = x + mixer(P.rms_norm(x, w[f"{p}.input_layernorm.weight"], eps))
            x = x + P.swiglu_mlp(P.rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], eps), w, f"{p}.mlp")
        return P.linear(P.rms_norm(x, w["model.norm.weight"], eps), w["model.embed_tokens.weight"]).numpy()

    rng = np.random.default_rng(1)
    toks = {r: rng.integers(0, 1000, n).tolist() for r, n in (("a", 30), ("b", 21), ("c", 9))}
    got, fed = {r: {} for r in toks}, {r: 0 for r in toks}

    def run(parts, end=()):
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
        for r in end:
            cache.close(r)

    # portions beside single tokens; "c" runs in the pages that "b" gave back
    run([("a", 11)]); run([("a", 2), ("b", 9)]); run([("a", 1), ("b", 1)]); run([("b", 11), ("a", 16)], end=["b"])
    run([("c", 7)]); run([("c", 2)], end=["c", "a"])
    t = 2e-5 if dtype == "float32" else 3e-2
    for r in toks:
        want = plain(toks[r])
        have = np.stack([got[r][i] for i in range(len(toks[r]))])
        assert np.abs(have - want).max() / max(1.0, np.abs(want).max()) <= t, r
    cache.check_invariants()
    assert cache.available() == 12


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_is_captured_around_a_mixer_that_cannot_be(tmp_path, dtype):
    """The toy mixer with state loops over the step on the host (graph_safe is False).  The step is
    captured all the same: the capture ends before each such mixer and begins again behind it, and at
    every replay the mixer alone is launched between the captured pieces.  Three requests decode through
    the step captured for four (one row of padding), against the plain implementation."""
    register_mixer("running_mean", RunningMeanMixer, replace=True)
    register_architecture(Architecture("ToyStateForCausalLM", parse=parse_toy, describe=describe_toy), replace=True)
    model = write_random_model(str(tmp_path / "toy"), TOY, 3)
    runner = ModelRunner(model, dtype=dtype, page_size=8, num_pages=24, max_requests=4)
    assert runner.use_graphs and runner.model.capturable()
    cache = runner.cache
    rng = np.random.default_rng(2)
    lens, steps = dict(a=19, b=3, c=30), 6
    toks = {r: rng.integers(0, 1000, n + steps).tolist() for r, n in lens.items()}
    for r, n in lens.items():
        cache.open(r)
        assert cache.reserve(r, n)
        runner.step([StepEntry(r, toks[r][:n], [])])
        cache.commit(r, n)
    want = {r: plain_toy(model, t) for r, t in toks.items()}
    zeros = np.zeros(3, dtype=np.float32)
    t = 2e-5 if dtype == "float32" else 3e-2
    for i in range(steps):
        entries = [StepEntry(r, [toks[r][lens[r] + i]], [0]) for r in lens]
        for r in lens:
            assert cache.reserve(r, 1)
        logits, tokens = runner.step_and_sample(entries, zeros, zeros)
        logits = logits.cpu().numpy()
        graph = runner._decode_graph(entries)
        kinds = [p[0] for p in graph.pieces]
        # layers 0, toy, 0 again, toy: graph, toy, graph, toy, graph
        assert graph.B == 4 and kinds == ["graph", "eager", "graph", "eager", "graph"]
        runner.check_status()
        assert (tokens.cpu().numpy()[1:] == logits.argmax(1)).all()
        for row, r in enumerate(lens):
            w = want[r][lens[r] + i]
            assert np.abs(logits[row] - w).max() / max(1.0, np.abs(w).max()) <= t, (r, i)
        for r in lens:
            cache.commit(r, 1)
    for r in lens:
        cache.close(r)
    cache.check_invariants()
