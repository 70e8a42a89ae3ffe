"""The cache manager without a device: the allocator's order of handing out and
evicting (crates/pagedllm/src/blocks.rs:432-675 has the reference's cases),
tables, groups, windows, sharing, state slots, and no page lost, held twice or
freed twice under random orders of requests."""

import random

import pytest
import torch

from paged_llm_rs_b200.cache import BlockAllocator, CacheManager, FREED, block_hash
from paged_llm_rs_b200.errors import CacheError
from paged_llm_rs_b200.parts.base import KVNeed, StateNeed

FULL = KVNeed("full", 2, 16)
WIN = KVNeed("window", 2, 16, window=20)


def manager(needs, pages, page_size=4, max_requests=8, prefix=True):
    return CacheManager(needs, page_size, pages, max_requests, torch.float32, "cpu", prefix_cache=prefix,
                        allocate_device=False)


def test_hash_chains_on_the_parent():
    a = block_hash(None, [1, 2, 3, 4])
    assert a == block_hash(None, [1, 2, 3, 4]) and a != block_hash(None, [1, 2, 3, 5])
    assert block_hash(a, [5, 6]) != block_hash(None, [5, 6])          # same tokens after another prefix
    assert block_hash(None, [1, 2]) != block_hash(None, [1, 2, 0])    # the length is part of the name
    assert 0 <= a < 2 ** 64


def test_allocator_hands_out_zero_first_and_unnamed_pages_before_named():
    a = BlockAllocator(4)
    assert [a.allocate() for _ in range(4)] == [0, 1, 2, 3] and a.allocate() is None
    a.publish(1, 111)
    a.publish(2, 222)
    for b in (1, 2, 0):   # released in this order: 1 is the longest unheld of the named ones
        a.release(b)
    assert a.allocate() == 0 and a.evictions == 0     # the page without a name goes first
    assert a.allocate() == 1 and a.evictions == 1     # then the named page released longest ago
    assert a.acquire_cached(111) is None and a.acquire_cached(222) == 2   # 2 kept its name and is held again
    assert a.available() == 0
    a.check()


def test_allocator_first_owner_keeps_a_name_and_double_release_is_an_error():
    a = BlockAllocator(3)
    x, y = a.allocate(), a.allocate()
    a.publish(x, 7)
    a.publish(y, 7)
    assert a.acquire_cached(7) == x and a.holders(x) == 2
    a.release(x); a.release(x)
    with pytest.raises(CacheError):
        a.release(x)
    with pytest.raises(CacheError):
        a.release(99)
    a.clear_cache()
    assert a.acquire_cached(7) is None


def test_tables_slots_and_reserve_is_all_or_nothing():
    m = manager([FULL, WIN, FULL], pages=3)
    assert len(m.groups) == 2 and m.groups[0].entries == [0, 2] and m.groups[1].entries == [1]
    m.open("a")
    assert m.reserve("a", 9) and m.available() == 0       # 3 pages of 4 in both groups
    m.open("b")
    assert not m.reserve("b", 1)
    m.check_invariants()
    assert m.get("a").tables[0].slot_of(5) == m.get("a").tables[0].blocks[1] * 4 + 1
    m.commit("a", 9)
    with pytest.raises(CacheError):
        m.commit("a", 4)                                    # past what was reserved
    m.close("a")
    with pytest.raises(CacheError):
        m.close("a")                                        # closed twice
    assert m.available() == 3
    # one group dry, the other not: nothing stays taken
    m2 = manager([FULL, WIN], pages=2)
    m2.open("x")
    m2.groups[1].allocator.allocate()
    assert not m2.reserve("x", 8) and m2.groups[0].allocator.available() == 2
    assert m2.reserve_up_to("x", 8) == 4


def test_window_group_gives_pages_back_and_they_are_used_again():
    m = manager([WIN], pages=8, page_size=4)   # window 20: a query sees 20 keys
    m.open("a")
    seen = set()
    for step in range(30):
        assert m.reserve("a", 3), step
        seen.update(b for b in m.get("a").tables[0].blocks if b >= 0)
        m.commit("a", 3)
        t = m.get("a").tables[0]
        first_needed = max(0, t.tokens - 20 + 1)
        for i, b in enumerate(t.blocks):
            assert (b == FREED) == ((i + 1) * 4 <= first_needed)
        m.check_invariants()
    assert m.tokens_of("a") == 90 and len(seen) <= 8      # 23 logical pages went through at most 8 physical ones
    assert m.groups[0].allocator.in_use() <= 7
    m.close("a")
    assert m.available() == 8


def test_prefix_is_shared_but_never_the_last_page():
    m = manager([FULL], pages=8, page_size=4)
    prompt = list(range(12))
    m.open("a"); assert m.claim_prefix("a", prompt) == 0
    m.reserve("a", 12); m.commit("a", 12, prompt)
    m.open("b")
    assert m.claim_prefix("b", prompt) == 8                 # two full pages, the third is left alone
    assert m.get("b").tables[0].blocks == m.get("a").tables[0].blocks[:2]
    m.open("c")
    assert m.claim_prefix("c", prompt[:4] + [99] * 8) == 4  # agrees for one page only
    m.open("d")
    assert m.claim_prefix("d", [99] * 4 + prompt[4:]) == 0  # same later tokens after another prefix
    m.check_invariants()
    m.close("a")
    m.check_invariants()
    assert m.groups[0].allocator.holders(m.get("b").tables[0].blocks[0]) == 2   # b and c still hold it
    for r in "bcd":
        m.close(r)
    m.open("e")
    assert m.claim_prefix("e", prompt) == 8                 # pages kept their names while unheld
    # windows and state switch sharing off
    assert not manager([FULL, WIN], 4).prefix_cache and not manager([FULL, StateNeed((4,))], 4).prefix_cache


def test_state_slots():
    m = CacheManager([FULL, StateNeed((3, 2))], 4, 4, 2, torch.float32, "cpu")
    state = m.layer_caches()[1]
    assert state.shape == (2, 3, 2)
    a = m.open("a").state_slot
    state[a] += 5
    b = m.open("b").state_slot
    assert a != b
    with pytest.raises(CacheError):
        m.open("c")
    m.close("a")
    assert m.open("c").state_slot == a and state[a].abs().sum() == 0   # zeroed for the new request
    m.check_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    rnd = random.Random(seed)
    needs = [[FULL], [FULL, WIN], [WIN, FULL, FULL]][seed % 3]
    m = manager(needs, pages=12, page_size=4, max_requests=5, prefix=seed % 2 == 0)
    live, histories, next_id = [], {}, 0
    for _ in range(600):
        op = rnd.random()
        if op < 0.25 and len(live) < 5:
            rid = next_id; next_id += 1
            m.open(rid); live.append(rid)
            histories[rid] = [rnd.randrange(3) for _ in range(rnd.randrange(1, 30))]
            shared = m.claim_prefix(rid, histories[rid])
            histories[rid] = histories[rid]  # tokens [0, shared) are already in the cache
            assert m.tokens_of(rid) == shared
        elif op < 0.8 and live:
            rid = rnd.choice(live)
            n = rnd.randrange(1, 9)
            got = m.reserve_up_to(rid, n) if rnd.random() < 0.5 else (n if m.reserve(rid, n) else 0)
            if got:
                done = m.tokens_of(rid)
                while len(histories[rid]) < done + got:
                    histories[rid].append(rnd.randrange(3))
                m.commit(rid, got, histories[rid])
        elif live:
            rid = live.pop(rnd.randrange(len(live)))
            m.close(rid)
        m.check_invariants()
    for rid in live:
        m.close(rid)
    m.check_invariants()
    assert all(g.allocator.available() == 12 for g in m.groups) and m.slots_free() == 5
