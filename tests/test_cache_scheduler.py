"""The cache manager and the scheduler's decisions (no GPU, no model)."""
import random

import pytest
import torch

from zig_ai_b200.cache import CacheManager, IdPool, OutOfPages
from zig_ai_b200.engine.scheduler import Request, RequestRefused, Scheduler
from zig_ai_b200.parts.base import PagedKVNeed, StateNeed
from zig_ai_b200.sampling import SamplingParams

FULL = PagedKVNeed(2, 16)
WIN = PagedKVNeed(2, 16, window=20)
STATE = StateNeed((2, 8))


def manager(needs, page_size=4, num_pages=16, max_requests=4):
    return CacheManager([("own", n) for n in needs], page_size, num_pages, max_requests, torch.float32, "cpu",
                        allocate=False)


def test_pool_refuses_misuse():
    p = IdPool(3, first=1)
    a, b, c = p.alloc(), p.alloc(), p.alloc()
    assert sorted([a, b, c]) == [1, 2, 3]
    with pytest.raises(OutOfPages):
        p.alloc()
    p.free(b)
    with pytest.raises(ValueError):
        p.free(b)                      # freed twice
    with pytest.raises(ValueError):
        p.free(99)
    assert p.alloc() == b
    p.check()


def test_groups_planes_and_shared_caches():
    needs = [("own", STATE), ("own", FULL), ("own", STATE), ("own", FULL), ("shared", 1), ("own", WIN)]
    m = CacheManager(needs, 4, 8, 2, torch.float32, "cpu")
    assert len(m.groups) == 3
    assert m.where == [[(0, 0)], [(1, 0)], [(0, 1)], [(1, 1)], [(1, 0)], [(2, 0)]]
    assert m.groups[1].data.shape == (2, 9, 2, 2, 4, 16) and m.groups[0].data.shape == (2, 3, 2, 8)
    assert m.bytes_per_token() == (2 + 1) * 2 * 2 * 16 * 4


def test_several_needs_per_layer_call_and_other_page_layouts():
    """A layer call may need pages and a state, or two states (a state matrix beside a conv state); a
    paged need may hold one vector per position instead of keys and values; a state may be kept in
    another dtype than 32-bit.  Each need gets a view of its own; equal needs share a group."""
    from zig_ai_b200.parts.base import PagedRowsNeed
    matrix, conv = StateNeed((4, 4), "bfloat16"), StateNeed((2, 8))
    latent = PagedRowsNeed(24)
    needs = [("own", (FULL, conv)), ("own", (matrix, conv)), ("own", None), ("own", latent), ("shared", 1), ("own", (latent, FULL))]
    m = CacheManager(needs, 4, 8, 2, torch.float32, "cpu")
    assert [type(g.need).__name__ for g in m.groups] == ["PagedKVNeed", "StateNeed", "StateNeed", "PagedRowsNeed"]
    assert m.where == [[(0, 0), (1, 0)], [(2, 0), (1, 1)], [], [(3, 0)], [(2, 0), (1, 1)], [(3, 1), (0, 1)]]
    assert m.groups[2].data.dtype == torch.bfloat16 and m.groups[2].data.shape == (1, 3, 4, 4)
    assert m.groups[3].data.shape == (2, 9, 4, 24)
    assert m.bytes_per_token() == (2 * 2 * 2 * 16 + 2 * 24) * 4

    class Step:
        block_tables = {0: "kv tables", 3: "latent tables"}
    v = m.views(5, Step)
    assert len(v) == 2 and v[0].block_table == "latent tables" and v[0].pages.shape == (9, 4, 24)
    assert v[1].block_table == "kv tables" and v[1].pages.shape == (9, 2, 2, 4, 16)
    assert m.views(2, Step) == [] and m.view(2, Step).pages is None and m.view(1, Step).state.shape == (3, 4, 4)
    # pages of both paged groups are taken and given back together
    m.admit("a")
    m.reserve("a", 9)
    assert m.groups[0].pool.n_used == 3 and m.groups[3].pool.n_used == 3
    m.release("a")
    m.check()


def test_pages_taken_returned_and_reused():
    m = manager([FULL, STATE])
    m.admit("a")
    m.reserve("a", 9)                  # 3 pages
    assert m.requests["a"].tables[0] == [1, 2, 3] and m.groups[0].pool.n_free == 13
    m.reserve("a", 10)                 # same page
    assert len(m.requests["a"].tables[0]) == 3
    m.admit("b")
    with pytest.raises(OutOfPages):
        m.reserve("b", 14 * 4)
    assert m.requests["b"].tables[0] == []          # nothing was taken
    m.release("a")
    m.reserve("b", 14 * 4)
    assert m.pages_reused == 3
    m.check()
    with pytest.raises(KeyError):
        m.release("a")                 # given back twice


def test_window_group_gives_pages_back_early():
    m = manager([WIN], page_size=4, num_pages=16)
    m.admit("a")
    total = 0
    for n in [3, 6, 1, 1, 9, 1, 1, 1, 30, 1, 1]:
        total += n
        m.reserve("a", total)
        t = m.requests["a"].tables[0]
        # every position a query of the next step may read still has its page
        first_needed = max(total - n - 20 + 1, 0)
        for p in range(first_needed, total):
            assert t[p // 4] > 0, (total, p)
        m.check()
    held = [p for p in m.requests["a"].tables[0] if p > 0]
    assert len(held) <= (20 + 30) // 4 + 2 and m.requests["a"].tables[0][0] == -1
    assert m.table_rows(["a"], 0, 20)[0][0] == 0     # a released page reads as the null page


def test_random_orders_lose_nothing():
    g = random.Random(0)
    m = manager([FULL, WIN, STATE], page_size=4, num_pages=24, max_requests=5)
    live, sizes = {}, {}
    for it in range(3000):
        r = g.random()
        if r < 0.25 and len(live) < 5:
            k = f"r{it}"
            m.admit(k)
            live[k] = 0
        elif r < 0.8 and live:
            k = g.choice(list(live))
            n = g.choice([1, 1, 1, 2, 5, 17])
            try:
                m.reserve(k, live[k] + n)
                live[k] += n
            except OutOfPages:
                before = {kk: list(v.tables[0]) for kk, v in m.requests.items()}
                assert before == {kk: list(v.tables[0]) for kk, v in m.requests.items()}
                victim = max(live, key=live.get)
                m.release(victim)
                del live[victim]
        elif live:
            k = g.choice(list(live))
            m.release(k)
            del live[k]
        m.check()
        assert m.slots.n_used == len(live)
    for k in list(live):
        m.release(k)
    m.check()
    assert all(m.groups[g_].pool.n_free == 24 for g_ in m.paged_groups()) and m.slots.n_free == 5
    assert m.pages_reused > 0


# ----------------------------------------------------------------------------- scheduler
def req(i, n_prompt, max_new=4, **kw):
    return Request(i, list(range(1, n_prompt + 1)), SamplingParams(temperature=0.0, max_new_tokens=max_new, **kw))


def run(s, steps=1000):
    """Drive the scheduler with a fake model that always 'samples' token 7; returns the plans."""
    plans = []
    while s.has_work() and len(plans) < steps:
        plan = s.schedule()
        plans.append(plan)
        s.commit(plan, {e.request.request_id: 7 for e in plan.entries if e.sample})
        s.cache.check()
    return plans


def test_portions_under_a_token_budget_and_decodes_first():
    m = manager([FULL, STATE], page_size=4, num_pages=64, max_requests=4)
    s = Scheduler(m, max_num_seqs=4, max_batched_tokens=8, max_model_len=256)
    a, b = req("a", 19, max_new=3), req("b", 5, max_new=3)
    s.add(a)
    s.add(b)
    plans = run(s)
    sizes = [[(e.request.request_id, len(e.tokens), e.sample) for e in p.entries] for p in plans]
    assert sizes[0] == [("a", 8, False)]
    assert sizes[1] == [("a", 8, False)]
    assert sizes[2] == [("a", 3, True), ("b", 5, True)]          # a's last portion beside b's whole prompt
    assert sizes[3] == [("a", 1, True), ("b", 1, True)]          # both decode
    assert all(p.n_tokens <= 8 for p in plans)
    assert a.output == [7, 7, 7] and b.output == [7, 7, 7] and a.finish_reason == "length"
    assert m.slots.n_used == 0 and m.groups[0].pool.n_used == 0


def test_decoding_requests_come_before_new_prompts():
    m = manager([FULL], page_size=4, num_pages=64, max_requests=4)
    s = Scheduler(m, max_num_seqs=4, max_batched_tokens=6, max_model_len=256)
    a = req("a", 2, max_new=5)
    s.add(a)
    s.commit(p := s.schedule(), {"a": 7})
    s.add(req("b", 20, max_new=2))
    plan = s.schedule()
    assert [(e.request.request_id, len(e.tokens)) for e in plan.entries] == [("a", 1), ("b", 5)]


def test_refusals():
    m = manager([FULL], page_size=4, num_pages=8, max_requests=2)
    s = Scheduler(m, 2, 16, max_model_len=64)
    with pytest.raises(RequestRefused):
        s.add(req("long", 60, max_new=10))           # beyond the model's length
    with pytest.raises(RequestRefused):
        s.add(req("big", 30, max_new=10))            # beyond the pool, even alone
    with pytest.raises(RequestRefused):
        s.add(Request("empty", [], SamplingParams()))
    s.add(req("ok", 28, max_new=5))                  # 32 cached positions at most: fits exactly


def test_admission_waits_for_slots_and_pages():
    m = manager([FULL, STATE], page_size=4, num_pages=6, max_requests=2)
    s = Scheduler(m, max_num_seqs=2, max_batched_tokens=64, max_model_len=64)
    for i, n in enumerate([10, 10, 3]):
        s.add(req(i, n, max_new=2))
    plan = s.schedule()
    # 10 tokens take 3 pages each: the first two fit (6 pages), the third waits for a slot
    assert [e.request.request_id for e in plan.entries] == [0, 1]
    assert [r.request_id for r in s.waiting] == [2]
    s.commit(plan, {0: 7, 1: 7})
    plans = run(s)
    assert all(r.finish_reason == "length" for r in [e.request for e in plans[-1].entries])
    assert m.groups[0].pool.n_used == 0


def test_out_of_pages_preempts_the_newest_and_recomputes():
    m = manager([FULL, STATE], page_size=4, num_pages=6, max_requests=3)
    s = Scheduler(m, max_num_seqs=3, max_batched_tokens=64, max_model_len=64)
    a, b = req("a", 11, max_new=8), req("b", 11, max_new=8)
    s.add(a)
    s.add(b)
    plans = run(s)
    assert s.n_preemptions >= 1
    first = next(p for p in plans if p.preempted)
    assert [r.request_id for r in first.preempted] == ["b"]       # the newest admitted goes, the oldest stays
    assert all(e.request.request_id != "b" for e in first.entries)
    # b comes back whole: prompt plus what it had produced, as one recomputed portion
    back = next(p for p in plans[plans.index(first) + 1:] if any(e.request is b for e in p.entries))
    e = next(e for e in back.entries if e.request is b)
    assert e.tokens[:11] == b.prompt and len(e.tokens) > 11 and e.sample
    assert a.output == [7] * 8 and b.output == [7] * 8 and b.preemptions >= 1
    assert m.groups[0].pool.n_used == 0 and m.slots.n_used == 0


def test_a_lone_request_that_cannot_grow_ends_with_out_of_pages():
    # a window group keeps few pages, but a full group of the same manager runs out
    m = manager([FULL], page_size=4, num_pages=3, max_requests=2)
    s = Scheduler(m, 2, 64, max_model_len=64)
    r = req("a", 10, max_new=3)                      # 12 cached positions: fits exactly
    s.add(r)
    run(s)
    assert r.finish_reason == "length"
    m2 = manager([FULL, WIN], page_size=4, num_pages=3, max_requests=2)
    s2 = Scheduler(m2, 2, 64, max_model_len=64)
    m2.groups[0].pool.alloc()                        # a page lost to someone else: the pool is now too small
    r2 = req("b", 10, max_new=3)
    s2.add(r2)
    plans = []
    while s2.has_work():
        p = s2.schedule()
        plans.append(p)
        s2.commit(p, {e.request.request_id: 7 for e in p.entries if e.sample})
    assert r2.finish_reason == "out_of_pages" and any(p.failed for p in plans)


def test_eos_and_model_length_stop():
    m = manager([FULL], page_size=4, num_pages=32, max_requests=2)
    s = Scheduler(m, 2, 64, max_model_len=12)
    a = req("a", 3, max_new=9, eos_id=7)
    s.add(a)
    run(s)
    assert a.output == [7] and a.finish_reason == "eos"
    b = req("b", 4, max_new=8)
    s.add(b)
    run(s)
    assert b.finish_reason == "length" and len(b.output) == 8


def test_random_workloads_always_finish_and_free_everything():
    g = random.Random(1)
    for trial in range(20):
        m = manager([FULL, WIN, STATE], page_size=4, num_pages=g.choice([8, 12, 30]), max_requests=g.choice([1, 2, 4]))
        s = Scheduler(m, max_num_seqs=4, max_batched_tokens=g.choice([1, 3, 16, 64]), max_model_len=64)
        reqs = []
        for i in range(g.randrange(1, 9)):
            r = req(i, g.randrange(1, 20), max_new=g.randrange(1, 10))
            try:
                s.add(r)
                reqs.append(r)
            except RequestRefused:
                pass
        plans = run(s, steps=5000)
        assert not s.has_work()
        for r in reqs:
            assert r.finish_reason == "length" and len(r.output) == r.params.max_new_tokens, (trial, r)
        assert m.slots.n_used == 0 and all(m.groups[gi].pool.n_used == 0 for gi in m.paged_groups())
