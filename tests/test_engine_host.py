"""The engine loop without a model or a GPU: a stand-in for the runner answers every
row with a constant token, fails where the test tells it to, and the loop's
bookkeeping is checked: a failed step ends exactly its own requests
(crates/pagedllm-server/src/engine.rs:338-348), their pages and state slots come
back, the others go on, and no step in flight outlives its requests."""

from types import SimpleNamespace

import pytest
import torch

from paged_llm_rs_b200.cache import CacheManager
from paged_llm_rs_b200.engine.engine import Engine
from paged_llm_rs_b200.engine.scheduler import Finish
from paged_llm_rs_b200.errors import KernelError
from paged_llm_rs_b200.parts.base import KVNeed, StateNeed


class StubRunner:
    """Steps like a ModelRunner: the token of every wanted row is ``token``.  Call number
    ``raise_at`` raises from the launch; call number ``bad_status_at`` comes back with a
    non-zero status word, as a kernel that met an index out of range leaves it."""

    def __init__(self, pages=32, page_size=4, needs=None, token=9, raise_at=None, bad_status_at=None):
        self.cache = CacheManager(needs or [KVNeed("full", 1, 16)], page_size, pages, 16, torch.float32, "cpu",
                                  prefix_cache=False, allocate_device=False)
        self.spec = SimpleNamespace(max_positions=4096)
        self.vocab_size, self.device = 100, torch.device("cpu")
        self.graph_step_tokens, self.tokens_host, self.bytes_h2d = None, None, 0
        self.token, self.raise_at, self.bad_status_at, self.calls, self.status = token, raise_at, bad_status_at, 0, 0
        self.seen = []

    def step_and_sample(self, entries, temperature, uniform, check=False):
        self.calls += 1
        self.seen.append([e.request_id for e in entries])
        for e in entries:                                     # what the real packer checks
            rc = self.cache.get(e.request_id)
            assert rc.tokens + len(e.tokens) <= rc.tables[0].capacity()
        if self.calls == self.raise_at:
            raise KernelError("the stand-in refuses this step")
        n = sum(len(e.want) for e in entries)
        self.status = 2 if self.calls == self.bad_status_at else 0
        tokens = torch.tensor([self.status] + [self.token] * n, dtype=torch.int32)
        return torch.zeros((n, self.vocab_size)), tokens

    def prepack_decode(self, entries, temperature):
        return None

    def check_status(self):
        if self.status:
            self.status = 0
            raise KernelError("a kernel met a cache slot outside the pool")


def engine(runner, **kw):
    return Engine(None, runner=runner, **dict(dict(max_batch=8, chunk=None), **kw))


@pytest.mark.parametrize("how", ["raise_at", "bad_status_at"])
def test_a_failed_step_ends_its_requests_and_only_those(how):
    # three prompts run whole, one a step; the second one's step fails
    r = StubRunner(**{how: 2})
    eng = engine(r)
    ids = [eng.submit([1 + i, 2, 3, 4, 5], max_tokens=3) for i in range(3)]
    outs = []
    while eng.scheduler.has_work():
        out = eng.step()
        assert out is not None
        outs.append(out)
        r.cache.check_invariants()
    assert eng.finish_reason(ids[1]) == Finish.ERROR and isinstance(eng.last_error, KernelError)
    assert eng.finish_reason(ids[0]) == Finish.LENGTH and eng.finish_reason(ids[2]) == Finish.LENGTH
    assert eng._seqs[ids[0]].output == [9, 9, 9] and eng._seqs[ids[2]].output == [9, 9, 9]
    assert eng._seqs[ids[1]].output == []
    assert (ids[1], Finish.ERROR) in outs[1].finished and outs[1].tokens == []
    assert not any(ids[1] in seen for seen in r.seen[2:])          # the failed request is in no later step
    assert r.cache.available() == 32 and r.cache.slots_free() == 16 and eng._inflight is None


def test_a_failed_decode_step_takes_down_every_row_of_it_and_the_rest_goes_on():
    r = StubRunner(raise_at=4, needs=[KVNeed("full", 1, 16), StateNeed((3,))])
    eng = engine(r)
    a = [eng.submit([1 + i, 2, 3], max_tokens=6) for i in range(2)]
    for _ in range(3):                 # two prompts, then one decode step of both
        eng.step()
    late = eng.submit([7, 7, 7, 7, 7, 7], max_tokens=2)
    # whole-prompt mode admits the newcomer first; then the decode step of the two residents fails
    while eng.scheduler.has_work():
        assert eng.step() is not None
        r.cache.check_invariants()
    reasons = [eng.finish_reason(i) for i in a + [late]]
    assert reasons.count(Finish.ERROR) in (1, 2) and Finish.LENGTH in reasons
    assert r.cache.available() == 32 and r.cache.slots_free() == 16


def test_a_failure_in_a_mixed_step_ends_the_decoding_rows_and_the_prompt_in_flight():
    r = StubRunner(raise_at=3, pages=64)
    eng = engine(r, chunk=6)
    first = eng.submit([1, 2, 3, 4], max_tokens=8)
    eng.step()                                               # its prompt, whole (4 of 6)
    second = eng.submit(list(range(1, 15)), max_tokens=2)    # 14 tokens: portions of 5 beside the decoding row
    eng.step()                                               # decode + portion
    out = eng.step()                                         # fails: both were in it
    assert sorted(out.finished) == sorted([(first, Finish.ERROR), (second, Finish.ERROR)])
    assert not eng.scheduler.has_work() and r.cache.available() == 64
    third = eng.submit([5, 6, 7], max_tokens=2)              # the engine goes on
    eng.run_until_done()
    assert eng.finish_reason(third) == Finish.LENGTH and eng._seqs[third].output == [9, 9]


def test_how_requests_ended_is_remembered_for_a_bounded_number_of_them():
    r = StubRunner(pages=64)
    eng = engine(r)
    eng.FINISH_MEMORY = 5
    ids = [eng.submit([1, 2], max_tokens=1) for _ in range(12)]
    eng.run_until_done()
    assert len(eng._finish) == 5 and eng.finish_reason(ids[-1]) == Finish.LENGTH and eng.finish_reason(ids[0]) is None
