"""The native packer of the decode step (csrc/step_pack.cu) against the Python packer it
stands in for (engine/step.py): the same buffer, word for word, and the same refusals."""

import numpy as np
import pytest
import torch

from paged_llm_rs_b200.cache.manager import CacheManager
from paged_llm_rs_b200.engine.step import GroupPlanConfig, NativeDecodePacker, StepCaps, StepEntry, StepPacker
from paged_llm_rs_b200.errors import CacheError, ConfigError
from paged_llm_rs_b200.kernels import attention_plan
from paged_llm_rs_b200.parts.base import KVNeed, RowNeed

FULL = KVNeed("full", 2, 16, None)
WIN = KVNeed("window", 1, 32, 300)
ROWS = RowNeed(24)          # a group whose mixer reads tables and slots only: no attention work items


def setup(needs, plans, pages, page_size, B, W, target):
    cache = CacheManager(needs, page_size, pages, 16, torch.float32, "cpu", prefix_cache=False, allocate_device=False)
    packer = StepPacker(cache, plans, target, vocab_size=1000, max_positions=5000, device="cpu")
    caps = StepCaps(tokens=B, wanted=B, segments=B, table_width=W)
    work_caps = [None if p is None else attention_plan.plan_limits(B, p.tile_tokens, target, p.ctas_per_item) for p in plans]
    host, layout, _ = packer.pack([], caps, work_caps)
    out = np.full(len(host), 7, dtype=np.int32)       # stale contents must not show through
    return cache, packer, caps, work_caps, NativeDecodePacker(packer, caps, work_caps, layout, out), out


@pytest.mark.parametrize("target", [1, 64, 296, 10 ** 5])
@pytest.mark.parametrize("needs,plans", [
    ([FULL], [GroupPlanConfig(8, 2, None)]),
    ([FULL, WIN], [GroupPlanConfig(8, 2, None), GroupPlanConfig(16, 1, 300)]),
    ([FULL, ROWS, WIN], [GroupPlanConfig(8, 4, None), None, GroupPlanConfig(16, 1, 300)]),
    ([ROWS], [None]),
])
def test_native_decode_packer_writes_what_the_python_packer_writes(needs, plans, target):
    rng = np.random.default_rng(target)
    B, W, ps = 8, 64, 16
    cache, packer, caps, work_caps, native, out = setup(needs, plans, 700, ps, B, W, target)
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
            want, _, _ = packer.pack(entries, caps, work_caps, t, u)
            native.pack(entries, t, u)
            assert np.array_equal(out, want), np.nonzero(out != want)[0][:10]
        for r in ids:
            cache.close(r)
    cache.check_invariants()


def test_native_decode_packer_refuses_like_the_python_packer():
    plans = [GroupPlanConfig(8, 2, None)]
    cache, packer, caps, work_caps, native, out = setup([FULL], plans, 100, 16, 4, 64, 296)
    cache.open("a")
    assert cache.reserve("a", 16)
    cache.commit("a", 16)                      # position 16 has no page yet
    for pack in (lambda e: packer.pack(e, caps, work_caps), lambda e: native.pack(e, None, None)):
        with pytest.raises(CacheError):
            pack([StepEntry("a", [1], [0])])
    assert cache.reserve("a", 1)
    for pack in (lambda e: packer.pack(e, caps, work_caps), lambda e: native.pack(e, None, None)):
        with pytest.raises(ConfigError):
            pack([StepEntry("a", [1000], [0])])        # token id outside the vocabulary
        with pytest.raises(ConfigError):
            pack([StepEntry("a", [1], [0])] * 5)       # more requests than the step holds
        pack([StepEntry("a", [999], [0])])
