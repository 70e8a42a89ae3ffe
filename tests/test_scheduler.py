"""The scheduler's decisions without a model (the reference's cases:
crates/pagedllm/src/scheduler.rs:803-1370).  Every row of a step is answered
with a constant token, as its ``step()`` helper does (scheduler.rs:826-830)."""

import pytest
import torch

from paged_llm_rs_b200.cache import CacheManager
from paged_llm_rs_b200.engine.scheduler import Finish, Plan, Scheduler, Sequence
from paged_llm_rs_b200.parts.base import KVNeed, StateNeed
from paged_llm_rs_b200.sampling import SamplingParams

GREEDY = SamplingParams.greedy()


def make(pages, page_size=4, max_batch=16, chunk=None, needs=None, max_requests=16, prefix=True, max_positions=None,
         max_prefill_seqs=1):
    cache = CacheManager(needs or [KVNeed("full", 1, 16)], page_size, pages, max_requests, torch.float32, "cpu",
                         prefix_cache=prefix, allocate_device=False)
    return Scheduler(cache, max_batch=max_batch, chunk=chunk, max_positions=max_positions,
                     max_prefill_seqs=max_prefill_seqs), cache


def seq(i, n, max_tokens=4, stop=(), start=0):
    return Sequence(i, [(start + k) % 50 + 1 for k in range(n)], GREEDY, max_tokens, stop)


def step(s, token=9):
    plan = s.plan()
    out = s.commit(plan, [token] * len(plan.ids))
    s.cache.check_invariants()
    return plan, out


def test_prompts_are_admitted_in_order_then_decoded_together():
    s, cache = make(pages=16)
    for i, n in enumerate((5, 3, 6)):
        s.submit(seq(i, n, start=10 * i))    # different tokens: nothing to share
    kinds = []
    for _ in range(3):
        plan, _ = step(s)
        kinds.append((plan.kind, plan.ids, [len(e.tokens) for e in plan.entries]))
    assert kinds == [("prefill", [0], [5]), ("prefill", [1], [3]), ("prefill", [2], [6])]
    plan, _ = step(s)
    assert plan.kind == "decode" and plan.ids == [0, 1, 2] and all(len(e.tokens) == 1 for e in plan.entries)
    assert s.metrics.prefills == 3 and s.metrics.decode_rows == 3


def test_pages_grow_one_at_a_time_and_a_stop_token_frees_them():
    s, cache = make(pages=8)
    s.submit(seq(0, 4, max_tokens=10, stop=[7]))
    step(s)                                 # prefill fills page 0 exactly
    assert cache.groups[0].allocator.in_use() == 1
    step(s)                                 # the first decode needs a second page
    assert cache.groups[0].allocator.in_use() == 2
    plan, out = step(s, token=7)            # the stop token ends it and is not returned
    assert out.tokens == [] and out.finished == [(0, Finish.STOP)]
    assert cache.available() == 8 and not s.has_work()


def test_max_tokens_ends_with_length():
    s, _ = make(pages=8)
    s.submit(seq(0, 3, max_tokens=2))
    outs = [step(s)[1] for _ in range(2)]
    assert [o.tokens for o in outs] == [[(0, 9)], [(0, 9)]] and outs[1].finished == [(0, Finish.LENGTH)]


def test_a_prompt_the_pool_can_never_hold_is_refused():
    s, cache = make(pages=2)
    s.submit(seq(0, 9))                     # needs 3 pages of 4
    s.submit(seq(1, 4))
    plan, out = step(s)
    assert plan.kind == "refused" and out.finished == [(0, Finish.LENGTH)]
    assert step(s)[0].ids == [1]


def test_admission_waits_for_pages():
    s, cache = make(pages=3)
    s.submit(seq(0, 8, max_tokens=1))
    s.submit(seq(1, 8, max_tokens=1))
    assert step(s)[0].ids == [0]            # takes 2 pages and finishes at once (max_tokens 1)
    assert step(s)[0].ids == [1]
    s.submit(seq(2, 8, max_tokens=50)); step(s)
    s.submit(seq(3, 8))
    before = s.metrics.admission_stalls
    plan, _ = step(s)                       # 1 page left: the newcomer stalls, the resident decodes
    assert plan.kind == "decode" and plan.ids == [2] and s.metrics.admission_stalls == before + 1


def test_pool_dry_evicts_the_newest_never_the_oldest():
    s, cache = make(pages=4)                # 16 tokens in all
    s.submit(seq(0, 7, max_tokens=50))
    s.submit(seq(1, 7, max_tokens=50, start=20))
    step(s); step(s)                        # both admitted: 2 pages each
    plan, _ = step(s)                       # token 8 fits in the second page
    assert plan.ids == [0, 1]
    plan, _ = step(s)                       # position 8 needs a third page: none left, the newest goes
    assert plan.kind == "decode" and plan.ids == [0]
    assert s.metrics.preemptions == 1 and [q.id for q in s.waiting] == [1]
    victim = s.waiting[0]
    assert victim.pending == victim.history and len(victim.history) == 9 and victim.preemptions == 1
    assert s.metrics.recomputed_tokens == 9
    # tokens already returned stay returned; it is recomputed from prompt plus output when room comes
    assert victim.output == [9, 9]
    for _ in range(40):
        if not s.has_work():
            break
        step(s)
    assert not s.has_work() and cache.available() == 4


def test_a_lone_request_that_outgrows_the_pool_stops_the_engine_not_the_process():
    s, cache = make(pages=1)
    s.submit(seq(0, 4, max_tokens=50))
    step(s)
    plan, out = step(s)                     # nobody else to evict: it ends with LENGTH instead of idling for good
    assert plan.kind == "outgrown" and out.finished == [(0, Finish.LENGTH)] and cache.available() == 1


def test_budget_covers_decodes_and_one_portion():
    s, cache = make(pages=64, chunk=8)
    for i in range(3):
        s.submit(seq(i, 2, max_tokens=50))
    for _ in range(3):
        step(s)
    assert len(s.running) == 3 and s.cache.available() == 61
    s.submit(seq(3, 19, max_tokens=50))
    plan, _ = step(s)                       # 3 decodes + 5 prompt tokens = 8
    assert plan.kind == "mixed" and plan.ids == [0, 1, 2]
    assert [len(e.tokens) for e in plan.entries] == [1, 1, 1, 5] and plan.entries[3].want == []
    assert plan.advanced[-1] == (3, 5)
    plan, _ = step(s)
    assert plan.entries[3].tokens == seq(3, 19).history[5:10]      # the portion goes on where the last ended
    plan, _ = step(s); plan, _ = step(s)                            # 15 done; 4 left
    assert [len(e.tokens) for e in plan.entries] == [1, 1, 1, 4] and plan.entries[3].want == [3]
    assert plan.ids == [0, 1, 2, 3]                                 # the last portion brings a token back
    assert s.metrics.mixed_steps == 7


def test_a_prompt_is_admitted_and_gets_a_portion_in_the_same_step():
    s, _ = make(pages=64, chunk=4)
    s.submit(seq(0, 6))
    plan, _ = step(s)
    assert plan.kind == "mixed" and plan.ids == [] and [len(e.tokens) for e in plan.entries] == [4]
    plan, _ = step(s)
    assert plan.ids == [0] and plan.entries[0].want == [1]


def test_one_prompt_in_flight_at_a_time():
    s, _ = make(pages=64, chunk=4)
    s.submit(seq(0, 10)); s.submit(seq(1, 3))
    for _ in range(2):
        plan, _ = step(s)
        assert [e.request_id for e in plan.entries] == [0]
    plan, _ = step(s)                       # request 0 finishes its prompt (2 left)
    assert [e.request_id for e in plan.entries] == [0] and plan.ids == [0]
    plan, _ = step(s)
    assert [e.request_id for e in plan.entries] == [0, 1] and [len(e.tokens) for e in plan.entries] == [1, 3]


def test_several_prompts_may_share_a_pass_when_asked():
    # three short prompts and a long one under a budget of 16: with max_prefill_seqs 3 the first
    # pass holds the three short ones whole; the long one starts in the next and, part-run, keeps
    # the following passes to itself; a decoded token rides along from the second pass on
    s, _ = make(pages=64, chunk=16, max_prefill_seqs=3)
    for i, n in enumerate((3, 5, 4, 30)):
        s.submit(seq(i, n, max_tokens=8, start=10 * i))
    plan, _ = step(s)
    assert [(e.request_id, len(e.tokens), list(e.want)) for e in plan.entries] == [(0, 3, [2]), (1, 5, [4]), (2, 4, [3])]
    assert plan.ids == [0, 1, 2]
    plan, _ = step(s)
    assert [(e.request_id, len(e.tokens)) for e in plan.entries] == [(0, 1), (1, 1), (2, 1), (3, 13)]
    assert plan.ids == [0, 1, 2]                      # the long prompt's portion wants no logits yet
    plan, _ = step(s)
    assert [(e.request_id, len(e.tokens)) for e in plan.entries] == [(0, 1), (1, 1), (2, 1), (3, 13)]
    plan, _ = step(s)
    assert [(e.request_id, len(e.tokens)) for e in plan.entries] == [(0, 1), (1, 1), (2, 1), (3, 4)]
    assert plan.ids == [0, 1, 2, 3]
    # the budget bounds the pass: two prompts of 10 under 16 tokens are 10 + 6, then 4
    s, _ = make(pages=64, chunk=16, max_prefill_seqs=4)
    s.submit(seq(0, 10)); s.submit(seq(1, 10, start=20))
    plan, _ = step(s)
    assert [(e.request_id, len(e.tokens), list(e.want)) for e in plan.entries] == [(0, 10, [9]), (1, 6, [])]
    plan, _ = step(s)
    assert [(e.request_id, len(e.tokens), list(e.want)) for e in plan.entries] == [(0, 1, [0]), (1, 4, [3])]


def test_mixed_step_gives_way_to_preemption_when_a_resident_needs_a_page():
    s, cache = make(pages=4, chunk=8)
    s.submit(seq(0, 8, max_tokens=50))
    step(s)
    s.submit(seq(1, 7, max_tokens=50, start=20))
    step(s)                                  # request 0 takes a third page for position 8, request 1 starts
    assert [e.request_id for e in s.plan().entries] == [0]     # no page for the rest of the prompt: 0 decodes alone
    for _ in range(4):
        step(s)
    # position 12 of request 0 needs a page: the half-run prompt is the newest and gives its pages back
    assert s.metrics.preemptions == 1 and [q.id for q in s.running] == [0] and [q.id for q in s.waiting] == [1]
    assert s.waiting[0].pending == s.waiting[0].history and s.waiting[0].prompt_left == 0


def test_portion_shrinks_to_the_pages_that_are_left():
    s, cache = make(pages=3, chunk=16)
    s.submit(seq(0, 4, max_tokens=50)); step(s)
    s.submit(seq(1, 12, max_tokens=2))
    plan, _ = step(s)                        # request 0 takes a page for position 4, one page is left
    assert [len(e.tokens) for e in plan.entries] == [1, 4] and plan.advanced[-1] == (1, 4)


def test_prefix_hits_are_counted_and_skip_the_shared_tokens():
    s, cache = make(pages=32, chunk=None)
    s.submit(seq(0, 12, max_tokens=1)); step(s)
    s.submit(seq(1, 12, max_tokens=1))       # the same 12 tokens
    plan, _ = step(s)
    assert [len(e.tokens) for e in plan.entries] == [4]      # two pages shared, the last page its own
    assert s.metrics.cached_tokens == 8 and s.metrics.prefilled_tokens == 16
    assert s.metrics.prefix_hit_rate() == pytest.approx(8 / 24)
    s2, _ = make(pages=32, chunk=None, prefix=False)
    s2.submit(seq(0, 12, max_tokens=1)); step(s2)
    s2.submit(seq(1, 12, max_tokens=1))
    assert [len(e.tokens) for e in step(s2)[0].entries] == [12]


def test_cancel_frees_waiting_and_running():
    s, cache = make(pages=8)
    s.submit(seq(0, 5, max_tokens=50)); s.submit(seq(1, 5, max_tokens=50))
    step(s)
    s.cancel(1)
    assert not s.waiting
    s.cancel(0)
    assert not s.running and cache.available() == 8


def test_max_batch_caps_decode_rows():
    s, _ = make(pages=64, max_batch=2)
    for i in range(3):
        s.submit(seq(i, 2, max_tokens=50))
    for _ in range(3):
        step(s)
    assert step(s)[0].ids == [0, 1]


def test_context_ends_at_the_last_position():
    s, _ = make(pages=64, max_positions=6)
    s.submit(seq(0, 4, max_tokens=50))
    outs = [step(s)[1] for _ in range(2)]
    assert outs[1].finished == [(0, Finish.LENGTH)]          # 6 tokens seen: the next would sit at position 6
    s.submit(seq(1, 7))
    assert step(s)[0].kind == "refused"


def test_state_slots_limit_admission_and_come_back_on_preemption():
    s, cache = make(pages=64, needs=[KVNeed("full", 1, 16), StateNeed((2,))], max_requests=2, chunk=8)
    for i in range(3):
        s.submit(seq(i, 2, max_tokens=6, start=10 * i))
    for _ in range(3):
        step(s)
    assert len(s.running) == 2 and len(s.waiting) == 1 and s.metrics.admission_stalls >= 1
    for _ in range(10):
        step(s)
    assert not s.has_work() and cache.slots_free() == 2


def test_window_model_runs_a_long_prompt_through_few_pages():
    win = KVNeed("window", 1, 16, window=8)
    s, cache = make(pages=6, needs=[win], chunk=4)
    s.submit(seq(0, 40, max_tokens=5))       # 10 pages of tokens through a pool of 6
    produced = []
    for _ in range(30):
        if not s.has_work():
            break
        produced += step(s)[1].tokens
    assert len(produced) == 5 and cache.available() == 6


def test_the_decode_step_after_a_decode_step_is_known_before_that_one_is_committed():
    # what the engine asks while a decode step runs: the same requests again, pages for one more token
    # each reserved; not when someone waits, a prompt is in flight, a request has ended or the pool is dry
    s, cache = make(pages=16, page_size=4, chunk=8)
    for i, n in enumerate((3, 4)):
        s.submit(seq(i, n, max_tokens=6, start=10 * i))
    while s.waiting or any(q.prompt_left for q in s.running):
        step(s)
    plan = s.plan()
    assert plan.kind == "decode" and plan.ids == [0, 1]
    before = cache.groups[0].allocator.in_use()
    seqs = s.continuation(plan)                      # request 1 stands at 4 committed: tokens 5 and 6 need page 2
    assert [q.id for q in seqs] == [0, 1]
    assert all(cache.blocks_needed(q.id, 2) == 0 for q in seqs) and cache.groups[0].allocator.in_use() >= before
    cache.check_invariants()
    assert not s.ends_with(seqs[0], 9) and s.ends_with(seqs[0], 9) is False
    stopper = Sequence(7, [1, 2], GREEDY, 5, [9])
    assert s.ends_with(stopper, 9) and not s.ends_with(stopper, 8)
    stopper.generated = 4
    assert s.ends_with(stopper, 8)                   # the budget's last token
    steps, rows = s.metrics.steps, s.metrics.decode_rows
    s.count_decode_step(2)
    assert (s.metrics.steps, s.metrics.decode_rows) == (steps + 1, rows + 2)
    s.commit(plan, [9, 9])
    cache.check_invariants()
    # someone waits: the next step is a mixed one
    plan = s.plan()
    s.submit(seq(5, 3))
    assert s.continuation(plan) is None
    s.commit(plan, [9, 9])
    # a prompt in flight
    plan = s.plan()
    assert plan.kind == "mixed" and s.continuation(plan) is None
    s.commit(plan, [9, 9, 9])


def test_no_continuation_from_a_dry_pool():
    s, cache = make(pages=2, page_size=4)
    s.submit(seq(0, 4, max_tokens=20))
    step(s)                                           # the prompt fills page 0
    plan = s.plan()                                   # the first decode takes page 1: positions 4 .. 7
    assert plan.kind == "decode" and s.continuation(plan) is not None
    s.commit(plan, [9])
    for _ in range(2):
        step(s)                                       # 7 tokens committed
    plan = s.plan()                                   # position 7: fits; the one after it needs a third page
    assert plan.kind == "decode" and s.continuation(plan) is None
    s.commit(plan, [9])
    cache.check_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_random_traffic_with_steps_planned_ahead_loses_no_page(seed):
    # requests of random lengths, budgets and stop tokens arrive at random times, some are cancelled; the
    # driver does what the engine does (a decode step that follows a decode step is taken from
    # continuation() before the one before it is committed).  After every commit the books balance, and in
    # the end every page is free and every request got what its budget and its stop token allow.
    import random
    rng = random.Random(seed)
    chunk = rng.choice([None, 6, 16])
    s, cache = make(pages=rng.choice([10, 14, 40]), page_size=4, max_batch=rng.choice([3, 8]), chunk=chunk,
                    max_positions=64)
    todo = [Sequence(i, [rng.randrange(1, 50) for _ in range(rng.randrange(1, 14))], GREEDY, rng.randrange(1, 12),
                     [rng.choice([3, 77])]) for i in range(14)]
    seqs = {q.id: q for q in todo}
    produced, ahead, used_ahead, guard = {}, None, 0, 0
    while todo or s.has_work():
        guard += 1
        assert guard < 2000
        while todo and rng.random() < 0.4:
            s.submit(todo.pop())
        if ahead is not None:
            plan, ahead = ahead, None
            used_ahead += 1
        else:
            plan = s.plan()
            if plan.kind == "idle":
                if not todo:
                    assert not s.has_work() or s.waiting
                    if s.waiting:      # a prompt that waits for pages that will never come cannot happen here:
                        raise AssertionError("idle with requests waiting and nobody running")
                    break
                continue
            if plan.kind in ("refused", "outgrown"):
                s.commit(plan, [])
                cache.check_invariants()
                continue
        tokens = [rng.randrange(1, 6) for _ in plan.ids]
        # while the step "runs": the next one, if it is sure to be the same rows again
        nxt = s.continuation(plan)
        cache.check_invariants()
        if rng.random() < 0.05 and s.running:
            s.cancel(rng.choice(s.running).id)
            cache.check_invariants()
        goes_on = nxt is not None and not s.waiting and len(s.running) == len(plan.ids)
        if goes_on and not any(s.ends_with(q, t) for q, t in zip(nxt, tokens)):
            s.count_decode_step(len(nxt))
            ahead = Plan("decode", [q.id for q in nxt], [(q.id, 1) for q in nxt], [])
        out = s.commit(plan, tokens)
        cache.check_invariants()
        for rid, tok in out.tokens:
            produced.setdefault(rid, []).append(tok)
        if ahead is not None:
            # what the step planned ahead assumed still holds after the commit: the same requests, none ended,
            # each with its page for the token it will write
            assert [q.id for q in s.running] == ahead.ids
            assert all(q.finish is None and len(q.pending) == 1 and cache.blocks_needed(q.id, 1) == 0 for q in s.running)
    assert cache.available() == cache.num_pages
    cache.check_invariants()
    assert used_ahead > 0
    for q in seqs.values():
        got = produced.get(q.id, [])
        assert len(got) <= q.max_tokens and not (set(got) & q.stop_tokens)
        assert got == q.output
