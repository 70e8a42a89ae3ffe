"""The native packer of the decode step (csrc/step_pack.cu) against the Python packer it
stands in for (engine/step.py): the same buffer, word for word, and the same refusals."""

import numpy as np
import pytest
import torch

from paged_llm_rs_b200.cache.manager import CacheManager
from paged_llm_rs_b200.engine.step import GroupPlanConfig, NativeDecodePacker, StepCaps, StepEntry, StepPacker
from paged_llm_rs_b200.errors import CacheError, ConfigError
from paged_llm_rs_b200.kernels import attention_plan
from paged_llm_rs_b200.parts.base import KVNeed

FULL = KVNeed("full", 2, 16, None)
WIN = KVNeed("window", 1, 32, 300)


def setup(needs, plans, pages, page_size, B, W, target):
    cache = CacheManager(needs, page_size, pages, 16, torch.float32, "cpu", prefix_cache=False, allocate_device=False)
    packer = StepPacker(cache, plans, target, vocab_size=1000, max_positions=5000, device="cpu")
    caps = StepCaps(tokens=B, wanted=B, segments=B, table_width=W)
    work_caps = [attention_plan.plan_limits(B, p.tile_tokens, target, p.ctas_per_item) for p in plans]
    heads = [(4, 16)] * len(cache.groups)
    host, layout, _ = packer.pack([], heads, caps, work_caps)
    out = np.full(len(host), 7, dtype=np.int32)       # stale contents must not show through
    return cache, packer, caps, work_caps, heads, NativeDecodePacker(packer, caps, work_caps, layout, out), out


@pytest.mark.parametrize("target", [1, 64, 296, 10 ** 5])
@pytest.mark.parametrize("needs,plans", [
    ([FULL], [GroupPlanConfig(8, 2, None)]),
    ([FULL, WIN], [GroupPlanConfig(8, 2, None), GroupPlanConfig(16, 1, 300)]),
    ([FULL], [GroupPlanConfig(8, 2, None, 8)]),        # the kernel combines up to 8 items a token in a cluster
    ([FULL, WIN], [GroupPlanConfig(8, 4, None, 4), GroupPlanConfig(16, 1, 300)]),
])
def test_native_decode_packer_writes_what_the_python_packer_writes(needs, plans, target):
    rng = np.random.default_rng(target)
    B, W, ps = 8, 64, 16
    cache, packer, caps, work_caps, heads, native, out = setup(needs, plans, 700, ps, B, W, target)
    for trial in range(6):
        n = int(rng.integers(1, B + 1))
        ids = [f"r{trial}_{i}" for i in range(n)]
        for r in ids:
            ctx = int(rng.choice([0, 1, 15, 16, 17, 63, 64, 255, 256, 257, 600, 1000]))
            cache.open(r)
            assert cache.reserve(r, ctx + 1)
            cache.commit(r, ctx)
        entries = [StepEntry(r, [int(rng.integers(0, 1000))], [0]) for r in ids]
        temp = rng.random(n).astype(np.float32)
        uni = rng.random(n).astype(np.float32)
        for t, u in ((temp, uni), (None, None)):
            want, _, _ = packer.pack(entries, heads, caps, work_caps, t, u)
            native.pack(entries, t, u)
            assert np.array_equal(out, want), np.nonzero(out != want)[0][:10]
        for r in ids:
            cache.close(r)
    cache.check_invariants()


def test_native_decode_packer_refuses_like_the_python_packer():
    plans = [GroupPlanConfig(8, 2, None)]
    cache, packer, caps, work_caps, heads, native, out = setup([FULL], plans, 100, 16, 4, 64, 296)
    cache.open("a")
    assert cache.reserve("a", 16)
    cache.commit("a", 16)                      # position 16 has no page yet
    for pack in (lambda e: packer.pack(e, heads, caps, work_caps), lambda e: native.pack(e, None, None)):
        with pytest.raises(CacheError):
            pack([StepEntry("a", [1], [0])])
    assert cache.reserve("a", 1)
    for pack in (lambda e: packer.pack(e, heads, caps, work_caps), lambda e: native.pack(e, None, None)):
        with pytest.raises(ConfigError):
            pack([StepEntry("a", [1000], [0])])        # token id outside the vocabulary
        with pytest.raises(ConfigError):
            pack([StepEntry("a", [1], [0])] * 5)       # more requests than the step holds
        pack([StepEntry("a", [999], [0])])


@pytest.mark.parametrize("n,cpi,target,limit,expect", [
    (8, 8, 296, 8, 4), (4, 8, 296, 8, 8), (2, 8, 296, 8, 0), (16, 8, 296, 8, 2), (32, 8, 296, 8, 2), (64, 8, 296, 8, 0),
    (8, 8, 296, 0, 0), (8, 8, 296, 2, 2), (8, 8, 296, 1, 0), (1, 1, 296, 8, 0),
])
def test_cluster_size_of_a_decode_step(n, cpi, target, limit, expect):
    assert attention_plan.decode_cluster(n, cpi, target, limit) == expect


def test_cluster_plan_gives_every_token_whole_clusters_that_cover_its_keys():
    rng = np.random.default_rng(5)
    for C in (2, 3, 4, 8):
        pos = [int(p) for p in rng.choice([0, 1, 62, 63, 64, 65, 255, 256, 511, 512, 1000, 4095, 4096, 20000], size=9)]
        segs = [(i, 1, p) for i, p in enumerate(pos)]
        work, red, parts = attention_plan.plan_attention(segs, 8, None, 8, 296, cluster=C)
        assert len(red) == 0 and parts == 0 and len(work) == C * len(segs)
        for i, p in enumerate(pos):
            items = work[C * i:C * i + C]
            assert (items[:, 0] == i).all() and (items[:, 1] == i).all() and (items[:, 2] == 1).all() and (items[:, 3] == p).all()
            assert (items[:, 6] == -1).all() and list(items[:, 7]) == [(C << 16) | k for k in range(C)]
            assert (items[:, 4] % 64 == 0).all()                # every range starts on a key tile, the empty ones too
            live = items[items[:, 5] > items[:, 4]]
            assert live[0, 4] == 0 and live[-1, 5] == p + 1     # the keys 0 .. p, each once, in order
            assert (live[1:, 4] == live[:-1, 5]).all()
            assert len(live) == max(1, min(C, (p + 1) // attention_plan.MIN_SPLIT_KEYS)) or len(live) < C
            empty = items[items[:, 5] == items[:, 4]]
            assert len(live) + len(empty) == C and (items[:len(live)] == live).all()   # the live ones come first
    with pytest.raises(ValueError):
        attention_plan.plan_attention([(0, 2, 10)], 8, None, 8, 296, cluster=4)


def _covers(work, segs, tile):
    """Every query token's keys 0 .. its position, each once, over the items that hold the token."""
    seen = {}
    for seg, q0, qn, p0, kb, ke, part, split in work.tolist():
        for t in range(qn):
            lo, hi = kb, min(ke, p0 + t + 1)
            if hi > lo:
                seen.setdefault(q0 + t, []).append((lo, hi))
    for t0, n, p0 in segs:
        for t in range(n):
            runs = sorted(seen[t0 + t])
            assert runs[0][0] == 0 and runs[-1][1] == p0 + t + 1
            assert all(a[1] == b[0] for a, b in zip(runs, runs[1:]))


def test_tiles_of_many_tokens_are_cut_only_where_the_parts_stay_long():
    # one decoded token at 4095 beside a 512-token portion behind 1024 tokens: the single token is cut,
    # the portion's tiles (1088 .. 1536 keys) are not; the same portion behind 15 000 tokens is
    segs = [(0, 1, 4095), (1, 512, 1024)]
    work, red, parts = attention_plan.plan_attention(segs, 64, None, 8, 296)
    _covers(work, segs, 64)
    single, multi = work[work[:, 2] == 1], work[work[:, 2] > 1]
    assert len(single) == 4 and (single[:, 6] >= 0).all()          # 296 // (9 x 8) = 4 parts
    assert len(multi) == 8 and (multi[:, 6] == -1).all() and (multi[:, 7] == 0).all()
    assert len(red) == 1 and parts == 4
    segs = [(0, 1, 4095), (1, 512, 15000)]
    work, red, parts = attention_plan.plan_attention(segs, 64, None, 8, 296)
    _covers(work, segs, 64)
    multi = work[work[:, 2] > 1]
    assert len(multi) == 8 * 4 and (multi[:, 6] >= 0).all()
    assert ((multi[:, 5] - multi[:, 4]) >= attention_plan.MULTI_MIN_SPLIT_KEYS).all()
    assert len(red) == 1 + 512
    lim = attention_plan.plan_limits(513, 64, 296, 8, 2)
    assert len(work) <= lim[0] and len(red) <= lim[1] and parts <= lim[2]
