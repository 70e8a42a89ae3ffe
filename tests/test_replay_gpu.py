"""Trace replay against the plain implementation: the same requests whole, with
the last 32 tokens decoded one by one, in portions of changing size, and mixed
with other requests in a pool so small that pages are used again; long decoding;
the first tokens of a sequence; requests that share pages with equal prefixes;
and the same work as captured and replayed CUDA graphs, the way generation runs
it.  In float32 and in bfloat16, for two tiny configurations that differ in every
size and option (A on pages of 16; B, with a single kv head, on pages of 8), and
for two more with a window on some of their layers (W, D)."""

import numpy as np
import pytest

from tiny_configs import CONFIGS, PAGE_SIZES, write_model
from trace_tools import TraceBuilder, plain_logits, replay

pytestmark = pytest.mark.gpu

# worst |got - want| / max(1, max |want|), the reference's measure
# (crates/pagedllm/tests/common/mod.rs:20-43).  float32: observed 5e-7 on these
# models; bfloat16: 8 mantissa bits through a few layers, observed 6e-3.
TOL = {"float32": 2e-5, "bfloat16": 3e-2}
# the same position computed under another cut may differ by rounding only
TOL_CUT = {"float32": 2e-5, "bfloat16": 2e-2}

LENGTHS = {"w": 100, "d": 100, "c": 100, "long": 330, "f1": 1, "f2": 2, "f3": 3}


def tokens_for(name, vocab, n, seed):
    return np.random.default_rng([seed, sum(map(ord, name))]).integers(0, vocab, n).tolist()


def build_trace(vocab, seed):
    tb = TraceBuilder()
    toks = {k: tokens_for(k if k not in "wdc" else "same", vocab, n, seed) for k, n in LENGTHS.items()}
    # each request alone and whole
    tb.step([("w", toks["w"], range(100))], end=["w"])
    # most of it in one step, the last 32 tokens one by one
    tb.step([("d", toks["d"][:68], [67])])
    for i in range(68, 100):
        tb.step([("d", [toks["d"][i]], [0])], end=["d"] if i == 99 else [])
    # portions of changing size, down to two tokens, across page edges
    p = 0
    for n in (7, 2, 5, 3, 2, 16, 17, 2, 31, 15):
        tb.step([("c", toks["c"][p:p + n], range(n))], end=["c"] if p + n == 100 else [])
        p += n
    # the first tokens of a sequence
    for k in ("f1", "f2", "f3"):
        tb.step([(k, toks[k], range(len(toks[k])))])
    for k in ("f1", "f2", "f3"):
        tb.step([(k, [5], [0])], end=[k])
    # long decoding: 10 tokens whole, then 320 one by one
    tb.step([("long", toks["long"][:10], [9])])
    for i in range(10, 330):
        tb.step([("long", [toks["long"][i]], [0])], end=["long"] if i == 329 else [])
    toks["f1"], toks["f2"], toks["f3"] = toks["f1"] + [5], toks["f2"] + [5], toks["f3"] + [5]
    return tb, toks


def build_mixed(vocab, seed):
    """Six requests, at most four live, portions of some beside decoded tokens of
    others.  Every request is at most 64 tokens, so four live ones fit --max-tokens
    256 exactly: 16 pages of 16, and the later requests run in pages the earlier
    ones gave back."""
    rng = np.random.default_rng(seed + 100)
    lens = dict(m0=61, m1=37, m2=64, m3=50, m4=58, m5=33)
    toks = {k: rng.integers(0, vocab, n).tolist() for k, n in lens.items()}
    tb = TraceBuilder()
    fed = {k: 0 for k in lens}

    def portion(k, n, want_all=True):
        a = fed[k]
        n = min(n, lens[k] - a)
        fed[k] = a + n
        return (k, toks[k][a:a + n], range(n) if want_all else [n - 1])

    tb.step([portion("m0", 20), portion("m1", 9)])
    tb.step([portion("m0", 1), portion("m1", 2), portion("m2", 33)])
    tb.step([portion("m0", 1), portion("m2", 1), portion("m3", 17), portion("m1", 5)])
    while fed["m1"] < lens["m1"]:                  # m1 decodes to its end, the others go on in portions
        tb.step([portion("m1", 1), portion("m0", 1), portion("m3", 1), portion("m2", 1)],
                end=["m1"] if fed["m1"] == lens["m1"] else [])
    tb.step([portion("m4", 30, want_all=False), portion("m0", 1), portion("m3", 1)])   # m4 takes m1's pages
    while fed["m0"] < lens["m0"]:
        tb.step([portion("m0", 2), portion("m4", 1)], end=["m0"] if fed["m0"] == lens["m0"] else [])
    tb.step([portion("m5", 33), portion("m4", 4), portion("m2", 2)], end=["m5"])      # m5 in m0's pages
    for k in ("m2", "m3", "m4"):
        while fed[k] < lens[k]:
            tb.step([portion(k, 7)], end=[k] if fed[k] == lens[k] else [])
    return tb, toks


def err(got, want):
    return float(np.abs(got - want).max() / max(1.0, np.abs(want).max()))


PARAMS = [(n, d) for n in ("A", "B", "W", "D") for d in ("float32", "bfloat16")]


@pytest.fixture(scope="module", params=PARAMS, ids=lambda p: f"{p[0]}-{p[1]}")
def run(request, tmp_path_factory):
    name, dtype = request.param
    cfg, seed = CONFIGS[name]
    model = write_model(tmp_path_factory.mktemp("models"), name)
    V, ps = cfg["vocab_size"], PAGE_SIZES[name]
    tb, toks = build_trace(V, seed)
    got = tb.collect(replay(model, dtype, tb.steps, 640, V, page_size=ps))
    tbm, toksm = build_mixed(V, seed)
    gotm = tbm.collect(replay(model, dtype, tbm.steps, 256, V, page_size=ps))
    want = {k: plain_logits(model, t) for k, t in {**toks, **toksm}.items()}
    return dict(dtype=dtype, got={**got, **gotm}, want=want, name=name)


def rows(d, positions):
    return np.stack([d[p] for p in positions])


def test_whole_prompt_every_position(run):
    got = rows(run["got"]["w"], range(100))
    assert err(got, run["want"]["w"]) <= TOL[run["dtype"]]
    if run["dtype"] == "float32":
        assert (got.argmax(1) == run["want"]["w"].argmax(1)).all()


def test_last_32_tokens_one_by_one(run):
    got = rows(run["got"]["d"], range(67, 100))
    assert err(got, run["want"]["d"][67:]) <= TOL[run["dtype"]]
    assert err(got, rows(run["got"]["w"], range(67, 100))) <= TOL_CUT[run["dtype"]]


def test_portions_of_changing_size(run):
    got = rows(run["got"]["c"], range(100))
    assert err(got, run["want"]["c"]) <= TOL[run["dtype"]]
    assert err(got, rows(run["got"]["w"], range(100))) <= TOL_CUT[run["dtype"]]


def test_first_tokens_of_a_sequence(run):
    for k, n in (("f1", 1), ("f2", 2), ("f3", 3)):
        got = rows(run["got"][k], range(n + 1))
        assert err(got, run["want"][k]) <= TOL[run["dtype"]], k


def test_long_decoding(run):
    pos = list(range(9, 330))
    got = rows(run["got"]["long"], pos)
    assert err(got, run["want"]["long"][9:]) <= TOL[run["dtype"]]
    if run["dtype"] == "float32":
        assert (got.argmax(1) == run["want"]["long"][9:].argmax(1)).all()


def test_mixed_batches_in_reused_pages(run):
    for k in ("m0", "m1", "m2", "m3", "m4", "m5"):
        have = run["got"][k]
        pos = sorted(have)
        assert len(pos) >= 3, k
        assert err(rows(have, pos), run["want"][k][pos]) <= TOL[run["dtype"]], k


# --- as generation runs it: captured steps --------------------------------------------------------

def build_served(vocab, seed, budget):
    """Four requests as the scheduler would run them under a token budget, with given tokens
    instead of sampled ones: every step carries the next token of each request whose prompt
    is done (its logits wanted) and then one portion of the prompt in flight in the room
    that is left (the logits of its last token wanted when the prompt ends there).  Steps of
    single tokens replay the captured decode step (one, two, three and four requests: the
    step for four also runs with three, padded); portions that fill more than half of the
    budget replay the captured portion step; the rest are launched kernel by kernel."""
    rng = np.random.default_rng(seed + 200)
    prompt = dict(s0=90, s1=3, s2=130, s3=64)
    total = dict(s0=90 + 40, s1=3 + 70, s2=130 + 25, s3=64 + 33)
    toks = {k: rng.integers(0, vocab, n).tolist() for k, n in total.items()}
    tb = TraceBuilder()
    fed = {k: 0 for k in prompt}
    waiting, running = list(prompt), []
    while waiting or running:
        entries, room = [], budget
        for k in running:
            if fed[k] >= prompt[k]:
                entries.append((k, [toks[k][fed[k]]], [0]))
                room -= 1
        flying = [k for k in running if fed[k] < prompt[k]]
        if not flying and waiting:
            flying = [waiting.pop(0)]
            running.append(flying[0])
        if flying and room > 0:
            k = flying[0]
            n = min(room, prompt[k] - fed[k])
            entries.append((k, toks[k][fed[k]:fed[k] + n], [n - 1] if fed[k] + n == prompt[k] else []))
        for k, t, _ in entries:
            fed[k] += len(t)
        done = [k for k in running if fed[k] == total[k]]
        tb.step(entries, end=done)
        running = [k for k in running if k not in done]
    return tb, toks


@pytest.fixture(scope="module", params=PARAMS, ids=lambda p: f"{p[0]}-{p[1]}")
def served(request, tmp_path_factory):
    name, dtype = request.param
    cfg, seed = CONFIGS[name]
    model = write_model(tmp_path_factory.mktemp("models"), name)
    V, ps = cfg["vocab_size"], PAGE_SIZES[name]
    tb, toks = build_served(V, seed, 48)
    kinds = [("decode" if all(len(e["tokens"]) == 1 for e in s["entries"]) else "portion") for s in tb.steps]
    assert kinds.count("decode") >= 20 and kinds.count("portion") >= 6
    captured = tb.collect(replay(model, dtype, tb.steps, 640, V, page_size=ps, graphs=True, step_tokens=48))
    plain = tb.collect(replay(model, dtype, tb.steps, 640, V, page_size=ps))
    want = {k: plain_logits(model, t) for k, t in toks.items()}
    return dict(dtype=dtype, captured=captured, launched=plain, want=want)


def test_captured_steps_give_the_plain_implementations_logits(served):
    for k, have in served["captured"].items():
        pos = sorted(have)
        assert len(pos) >= 20, k
        assert err(rows(have, pos), served["want"][k][pos]) <= TOL[served["dtype"]], k
        if served["dtype"] == "float32":
            assert (rows(have, pos).argmax(1) == served["want"][k][pos].argmax(1)).all(), k


def test_captured_and_launched_steps_agree(served):
    for k, have in served["captured"].items():
        pos = sorted(have)
        assert sorted(served["launched"][k]) == pos
        assert err(rows(have, pos), rows(served["launched"][k], pos)) <= TOL_CUT[served["dtype"]], k


# --- equal prefixes share pages (crates/pagedllm/tests/prefix.rs) ------------------------------------

def build_shared(vocab, seed, ps):
    """The reference's cases on pages of ``ps`` tokens, every request alone and ended before the
    next starts, so that what it leaves behind is what the next one may take."""
    rng = np.random.default_rng(seed + 300)
    draw = lambda n: rng.integers(0, vocab, n).tolist()
    tb, toks, expect = TraceBuilder(), {}, {}

    def request(name, tokens, wanted, shares):
        toks[name], expect[name] = tokens, shares
        tb.step([(name, tokens, wanted)], end=[name])

    # the same prompt twice: the second takes every page but the last (prefix.rs:88-107)
    p = draw(50)
    request("same1", p, [49], 0)
    request("same2", p, [49], (50 - 1) // ps * ps)
    # a common head of 32 tokens, then different tails (prefix.rs:115-139)
    head = draw(32)
    request("tail_a", head + draw(18), range(40, 50), 0)
    request("tail_b", head + draw(18), range(40, 50), 32)
    # the same page of tokens after a different first page is another page (prefix.rs:146-170)
    middle = draw(ps)
    request("after_x", draw(ps) + middle + [7], [2 * ps], 0)
    request("after_y", draw(ps) + middle + [7], [2 * ps], 0)
    # ... also when the first page is found, which takes three prompts to reach (prefix.rs:182-223)
    head_a, head_c, mid = draw(ps), draw(ps), draw(ps)
    request("other", head_c + mid + [7], [2 * ps], 0)
    request("primer", head_a + draw(ps) + [7], [2 * ps], 0)
    request("under_test", head_a + mid + [7], [2 * ps], ps)
    return tb, toks, expect


@pytest.fixture(scope="module", params=[(n, d) for n in ("A", "B") for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def shared(request, tmp_path_factory):
    name, dtype = request.param
    cfg, seed = CONFIGS[name]
    model = write_model(tmp_path_factory.mktemp("models"), name)
    V, ps = cfg["vocab_size"], PAGE_SIZES[name]
    tb, toks, expect = build_shared(V, seed, ps)
    res = replay(model, dtype, tb.steps, 1024, V, page_size=ps, prefix_cache=True)
    want = {k: plain_logits(model, t) for k, t in toks.items()}
    return dict(dtype=dtype, got=tb.collect(res), prefix=res["prefix"], want=want, expect=expect, model=model, V=V, ps=ps)


def test_requests_take_the_pages_of_equal_prefixes_and_only_those(shared):
    assert shared["prefix"]["cached_tokens"] == shared["expect"]
    assert shared["prefix"]["hits"] == sum(shared["expect"].values()) // shared["ps"]
    assert shared["prefix"]["evictions"] == 0


def test_logits_over_shared_pages_are_those_of_the_plain_implementation(shared):
    for k, have in shared["got"].items():
        pos = sorted(have)
        assert err(rows(have, pos), shared["want"][k][pos]) <= TOL[shared["dtype"]], k
    same1, same2 = shared["got"]["same1"][49], shared["got"]["same2"][49]
    assert err(same2[None], same1[None]) <= TOL_CUT[shared["dtype"]]


def test_a_prompt_answers_the_same_after_its_pages_lost_their_names(shared):
    """prefix.rs:227-246: a pool that holds one prompt; a second prompt takes its pages and
    their names with them; the first prompt, run again, is computed anew."""
    V, ps = shared["V"], shared["ps"]
    rng = np.random.default_rng(77)
    p = rng.integers(0, V, 60).tolist()
    other = [(t + 50) % V for t in p]
    tb = TraceBuilder()
    tb.step([("first", p, [59])], end=["first"])
    tb.step([("other", other, [59])], end=["other"])
    tb.step([("again", p, [59])], end=["again"])
    res = replay(shared["model"], shared["dtype"], tb.steps, 64, V, page_size=ps, prefix_cache=True)
    got = tb.collect(res)
    assert res["prefix"]["evictions"] > 0
    assert res["prefix"]["cached_tokens"]["other"] == 0
    want = plain_logits(shared["model"], p)[59]
    for k in ("first", "again"):
        assert err(got[k][59][None], want[None]) <= TOL[shared["dtype"]], k
    assert err(got["again"][59][None], got["first"][59][None]) <= TOL_CUT[shared["dtype"]]


def test_trace_run_answers_step_by_step(tmp_path):
    """The protocol itself: a step may be sent only after `done <step>` of the one
    before; a step with nothing wanted writes no file; the program exits 0 at the
    end of its input."""
    import json, os, subprocess, sys
    from trace_tools import TRACE_RUN

    cfg, seed = CONFIGS["A"]
    model = write_model(tmp_path, "A")
    out = tmp_path / "out"
    p = subprocess.Popen([sys.executable, TRACE_RUN, "--model", model, "--dtype", "float32", "--out", str(out),
                          "--max-tokens", "64"], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    steps = [dict(step=0, entries=[dict(id="a", tokens=[1, 2, 3], want=[])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=[4, 5], want=[1])], end=["a"]),
             dict(step=2, entries=[dict(id="b", tokens=[1, 2, 3, 4, 5], want=[4])], end=["b"])]
    for s in steps:
        p.stdin.write(json.dumps(s) + "\n"); p.stdin.flush()
        assert p.stdout.readline().strip() == f"done {s['step']}"
    p.stdin.close()
    assert p.wait(timeout=60) == 0
    assert sorted(os.listdir(out)) == ["1.f32", "2.f32"]
    a = np.fromfile(out / "1.f32", dtype="<f4"); b = np.fromfile(out / "2.f32", dtype="<f4")
    assert a.shape == (cfg["vocab_size"],) and np.abs(a - b).max() <= 2e-5   # same tokens, other pages and cut
