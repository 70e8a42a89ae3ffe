"""The routes a decode step can take through the runner, compared at the level of
logits: launched kernel by kernel, replayed as the captured step (with fewer
requests than the step was captured for, so that some of it is padding), and
packed ahead of time and then replayed (what the engine does while the step before
runs).  The model is drawn so that attention decides the next token."""

import numpy as np
import pytest
import torch

import plain_qwen3 as P
from tiny_configs import CONFIGS, write_model

pytestmark = pytest.mark.gpu


def err(got, want):
    return float(np.abs(got - want).max() / max(1.0, np.abs(want).max()))


@pytest.mark.parametrize("name,dtype", [("D", "bfloat16"), ("D", "float32"), ("B", "bfloat16"), ("W", "bfloat16")])
def test_launched_captured_and_prepacked_steps_give_the_same_logits(tmp_path, name, dtype):
    from paged_llm_rs_b200.engine.runner import ModelRunner
    from paged_llm_rs_b200.engine.step import StepEntry

    cfg, seed = CONFIGS[name]
    model = write_model(tmp_path, name, decisive=True)
    V = cfg["vocab_size"]
    runner = ModelRunner(model, dtype=dtype, page_size=16, num_pages=64, max_requests=8, prefix_cache=False)
    cache = runner.cache
    rng = np.random.default_rng(seed + 40)
    lens = dict(a=70, b=5, c=131)          # three requests: the captured step for four runs with one row of padding
    steps = 12
    toks = {k: rng.integers(0, V, n + steps).tolist() for k, n in lens.items()}
    for k, n in lens.items():
        cache.open(k)
        assert cache.reserve(k, n)
        runner.step([StepEntry(k, toks[k][:n], [])])
        cache.commit(k, n)
    c64, w64 = P.load_model(model, torch.float64)
    want = {k: P.forward(c64, w64, toks[k]).numpy() for k in lens}
    # the plain model's next token depends on what attention adds (else this test could not see the cache)
    silent = {n: (v * 0 if "o_proj" in n else v) for n, v in w64.items()}
    moved = sum(int(P.forward(c64, silent, toks[k])[-1].argmax() != want[k][-1].argmax()) for k in lens)
    assert moved >= 2
    zeros = np.zeros(3, dtype=np.float32)
    tol = 2e-5 if dtype == "float32" else 3e-2
    worst_between = 0.0
    for i in range(steps):
        entries = [StepEntry(k, [toks[k][lens[k] + i]], [0]) for k in lens]
        for k in lens:
            assert cache.reserve(k, 2)      # this step's token and the next one's (the prepacked step stands one further)
        runner.use_graphs = False
        launched, _ = runner.step_and_sample(entries, zeros, zeros)
        launched = launched.cpu().numpy()
        runner.use_graphs = True
        captured, tokens = runner.step_and_sample(entries, zeros, zeros)
        captured, tokens = captured.cpu().numpy(), tokens.cpu().numpy()
        graph = runner._decode_graph(entries)
        assert graph.B == 4 and graph.native is not None
        runner.check_status()
        assert (tokens[1:] == captured.argmax(1)).all()
        worst_between = max(worst_between, err(captured, launched))
        for r, k in enumerate(lens):
            pos = lens[k] + i
            assert err(captured[r][None], want[k][pos][None]) <= tol, (k, i)
            assert err(launched[r][None], want[k][pos][None]) <= tol, (k, i)
            if dtype == "float32":
                assert captured[r].argmax() == want[k][pos].argmax()
        # the same step packed ahead of time: pack while the cache still counts one token less
        if i + 1 < steps:
            nxt = [StepEntry(k, [0], [0]) for k in lens]
            g2 = runner.prepack_decode(nxt, zeros)
            assert g2 is graph
            for k in lens:
                cache.commit(k, 1)
            feed = [toks[k][lens[k] + i + 1] for k in lens]
            ahead, _ = g2.launch_prepacked(feed, None)
            ahead = ahead.cpu().numpy().copy()
            again, _ = runner.step_and_sample([StepEntry(k, [t], [0]) for k, t in zip(lens, feed)], zeros, zeros)
            assert np.array_equal(ahead, again.cpu().numpy()), i      # the same captured kernels: bit for bit
        else:
            for k in lens:
                cache.commit(k, 1)
    assert worst_between <= (2e-5 if dtype == "float32" else 2e-2)
    runner.check_status()
    for k in lens:
        cache.close(k)
    cache.check_invariants()
