"""The scheduler's decisions (no GPU): budget, portions, admission order, preemption when pages run out."""
import pytest
import torch

from swifttransformer_b200.cache import CacheManager
from swifttransformer_b200.engine.scheduler import FINISHED, RUNNING, WAITING, Request, Scheduler
from swifttransformer_b200.parts.base import PagedKVSpec
from swifttransformer_b200.sampling import SamplingParams


def make(num_pages=64, page_size=4, max_seqs=8, budget=32, chunk=16, max_positions=200):
    cache = CacheManager([PagedKVSpec(1, 8)], torch.float32, "cpu", page_size, num_pages, max_seqs, max_positions)
    return cache, Scheduler(cache, budget, chunk, max_seqs, max_positions)


def req(i, n_prompt, max_new=4, **kw):
    return Request(i, list(range(3, 3 + n_prompt)), SamplingParams(max_new_tokens=max_new, **kw))


def run_step(sched, tok=7):
    plan = sched.schedule()
    done = sched.update(plan, [tok] * sum(1 for s in plan if s.samples))
    sched.cache.check()
    return plan, done


def test_budget_portions_and_order():
    cache, s = make(budget=32, chunk=16)
    for i, n in enumerate([40, 5, 30]):
        s.add(req(i, n))
    plan, _ = run_step(s)
    # first come first served: request 0 gets a full chunk, request 1 fits whole, request 2 gets what is left
    assert [(p.request.id, p.n) for p in plan] == [(0, 16), (1, 5), (2, 11)]
    assert sum(p.n for p in plan) <= 32
    assert [p.samples for p in plan] == [False, True, False]
    plan, _ = run_step(s)
    # decoding requests first (1 token), then running prompts in admission order, cut to the budget
    assert [(p.request.id, p.n) for p in plan] == [(1, 1), (0, 16), (2, 15)]
    plan, _ = run_step(s)
    assert [(p.request.id, p.n) for p in plan] == [(1, 1), (0, 8), (2, 4)]
    assert [p.samples for p in plan] == [True, True, True]
    plan, done = run_step(s)
    assert [(p.request.id, p.n) for p in plan] == [(0, 1), (1, 1), (2, 1)]   # all decoding, oldest first
    assert [r.id for r in done] == [1] and done[0].finish_reason == "length" and len(done[0].output) == 4
    while s.has_work():
        run_step(s)
    assert cache.free_pages == cache.total_pages and cache.num_free_slots == 8
    assert all(len(r.output) == 4 for r in s.finished)


def test_portion_down_to_one_token():
    cache, s = make(budget=9, chunk=8)
    s.add(req(0, 8))
    s.add(req(1, 6))
    plan, _ = run_step(s)
    assert [(p.request.id, p.n) for p in plan] == [(0, 8), (1, 1)]


def test_stop_conditions():
    cache, s = make(max_positions=12)
    s.add(req("eos", 4, max_new=10, eos_id=7))
    s.add(req("ign", 4, max_new=3, eos_id=7, ignore_eos=True))
    s.add(req("pos", 10, max_new=10))
    while s.has_work():
        run_step(s, tok=7)
    by = {r.id: r for r in s.finished}
    assert by["eos"].finish_reason == "eos" and by["eos"].output == [7]
    assert by["ign"].finish_reason == "length" and by["ign"].output == [7, 7, 7]
    # 10 prompt tokens + 2 generated reach the model's 12 positions: nothing more can be computed
    assert by["pos"].finish_reason == "positions" and len(by["pos"].output) == 2
    with pytest.raises(ValueError, match="positions"):
        s.add(req("long", 13))
    with pytest.raises(ValueError):
        s.add(Request("empty", [], SamplingParams()))


def test_preemption_when_pages_run_out():
    # 6 pages of 4 tokens; two requests of 8 prompt tokens fill 4 pages and then grow
    cache, s = make(num_pages=6, page_size=4, budget=64, chunk=64)
    s.add(req(0, 8, max_new=12))
    s.add(req(1, 8, max_new=12))
    seen_preempt = False
    steps = 0
    while s.has_work():
        plan, _ = run_step(s)
        steps += 1
        assert steps < 200
        if s.num_preemptions and not seen_preempt:
            seen_preempt = True
            # the request admitted last went back to the head of the queue, its tokens kept, its pages freed
            victim = s.waiting[0]
            assert victim.id == 1 and victim.state == WAITING and victim.n_computed == 0 and victim.slot is None
            assert len(victim.output) > 0
            assert s.running[0].id == 0
    assert seen_preempt
    by = {r.id: r for r in s.finished}
    assert len(by[0].output) == 12 and len(by[1].output) == 12
    assert by[1].preemptions >= 1 and by[0].preemptions == 0
    assert cache.free_pages == 6


def test_recompute_after_preemption_runs_prompt_and_output_as_one_prompt():
    cache, s = make(num_pages=5, page_size=4, budget=64, chunk=64)
    s.add(req(0, 8, max_new=8))
    s.add(req(1, 7, max_new=8))
    resumed = None
    for _ in range(100):
        if not s.has_work():
            break
        before = {r.id: len(r.output) for r in list(s.waiting) if r.preemptions}
        plan, _ = run_step(s)
        for p in plan:
            if p.request.id in before and resumed is None:
                resumed = (p.n, before[p.request.id])
    assert resumed is not None
    n, n_out = resumed
    assert n == 7 + n_out, "prompt and generated tokens are recomputed together"


def test_request_too_large_for_the_pool_is_finished_not_fatal():
    cache, s = make(num_pages=2, page_size=4, budget=64, chunk=64)
    s.add(req("big", 20))
    s.add(req("ok", 3, max_new=2))
    while s.has_work():
        run_step(s)
    by = {r.id: r for r in s.finished}
    assert by["big"].finish_reason == "cache_full" and by["big"].output == []
    assert by["ok"].finish_reason == "length" and len(by["ok"].output) == 2
    # a lone request that outgrows the pool while decoding
    cache, s = make(num_pages=2, page_size=4, budget=64, chunk=64)
    s.add(req("grow", 6, max_new=50))
    while s.has_work():
        run_step(s)
    r = s.finished[0]
    assert r.finish_reason == "cache_full" and len(r.output) == 3   # 6 + 3 tokens: the 9th has no page
    assert cache.free_pages == 2


def test_no_starvation_under_load():
    cache, s = make(num_pages=12, page_size=4, max_seqs=3, budget=16, chunk=8)
    for i in range(10):
        s.add(req(i, 5 + (i * 7) % 20, max_new=3 + i % 4))
    steps = 0
    while s.has_work():
        plan, _ = run_step(s)
        assert sum(p.n for p in plan) <= 16 and len({p.request.id for p in plan}) == len(plan)
        steps += 1
        assert steps < 500
    assert sorted(r.id for r in s.finished) == list(range(10))
    assert all(r.finish_reason == "length" for r in s.finished)


def test_update_in_two_halves_for_steps_launched_ahead():
    """update_pending + resolve: the next step can be decided before the tokens are known; a request that
    turns out to have ended is finished then, its later token is dropped and its pages come back."""
    from swifttransformer_b200.engine.scheduler import PENDING
    cache, s = make()
    s.add(req(0, 5, max_new=6, eos_id=9))
    s.add(req(1, 3, max_new=2))
    s.add(req(2, 4, max_new=6, eos_id=9, ignore_eos=True))
    plan1 = s.schedule()
    done, h1 = s.update_pending(plan1)
    assert done == [] and [r.output for r in s.running] == [[PENDING]] * 3
    plan2 = s.schedule()                                   # decided while plan1's tokens are unknown
    assert [(p.request.id, p.n, p.samples) for p in plan2] == [(0, 1, True), (1, 1, True), (2, 1, True)]
    done = s.resolve(h1, [9, 4, 9])                         # request 0 drew its end-of-sequence token
    assert [r.id for r in done] == [0] and done[0].output == [9] and done[0].finish_reason == "eos"
    assert s.running[0].output == [4] and s.running[1].output == [9]      # request 2 ignores it
    done, h2 = s.update_pending(plan2)                      # the step ahead: request 0's result is dropped
    assert h2[0] is None and [r.id for r in done] == [1] and done[0].finish_reason == "length"
    assert s.resolve(h2, [5, 6, 7]) == []
    assert done[0].output == [4, 6] and s.running[0].output == [9, 7]
    assert s.finished[0].output == [9]
    cache.check()
    while s.has_work():
        run_step(s)
    assert cache.free_pages == cache.total_pages
    with pytest.raises(ValueError):
        s.resolve([None], [])


@pytest.mark.parametrize("seed", range(12))
def test_invariants_under_random_load(seed):
    """Random pools, budgets, arrivals and lengths: a step never exceeds the token budget or the number of
    requests, names a request once, continues each request exactly where it stands, samples only at the end of
    what the request holds; requests arrive while others run; nothing is lost, every request ends with the tokens
    it was drawn (whatever was preempted in between), and the pool is whole again."""
    import random
    rnd = random.Random(seed)
    page = rnd.choice([2, 4, 8])
    max_seqs = rnd.randint(1, 6)
    budget = rnd.randint(4, 40)
    chunk = rnd.randint(1, budget)
    num_pages = rnd.randint(8, 40)
    cache, s = make(num_pages=num_pages, page_size=page, max_seqs=max_seqs, budget=budget, chunk=chunk, max_positions=120)
    todo = [(i, rnd.randint(1, 60), rnd.randint(1, 12)) for i in range(rnd.randint(3, 14))]
    drawn = {}                                   # request id -> tokens it was handed, in order
    steps = 0
    while todo or s.has_work():
        while todo and (not s.has_work() or rnd.random() < 0.4):
            i, n, m = todo.pop(0)
            s.add(req(i, n, max_new=m))
        plan = s.schedule()
        assert sum(p.n for p in plan) <= budget and len(plan) <= max_seqs
        assert len({p.request.id for p in plan}) == len(plan)
        for p in plan:
            r = p.request
            assert r.state == RUNNING and p.n >= 1 and r.n_computed + p.n <= len(r.tokens)
            assert p.samples == (r.n_computed + p.n == len(r.tokens))
            assert cache.lengths[r.slot] == r.n_computed
        toks = []
        for p in plan:
            if p.samples:
                t = 1000 * p.request.id + len(p.request.output)      # a token that says whose it is and which
                drawn.setdefault(p.request.id, []).append(t)
                toks.append(t)
        # the step "runs": pages for its tokens exist, lengths move on
        for p in plan:
            assert cache.reserve(p.request.slot, p.request.n_computed, p.request.n_computed + p.n)
            cache.commit(p.request.slot, p.request.n_computed + p.n)
        s.update(plan, toks)
        cache.check()
        steps += 1
        assert steps < 5000
    assert cache.free_pages == cache.total_pages and cache.num_free_slots == max_seqs
    assert len(s.finished) == len(drawn) + sum(1 for r in s.finished if not r.output)
    for r in s.finished:
        # the tokens a request keeps in the cache: all but the one drawn last
        fits_alone = len(r.prompt) + r.params.max_new_tokens - 1 <= num_pages * page
        assert (r.finish_reason == "cache_full") == (not fits_alone), (r.id, r.finish_reason, len(r.prompt))
        if fits_alone:
            assert r.finish_reason == "length" and r.output == drawn[r.id]
        else:
            assert r.output == drawn.get(r.id, [])


def test_a_newcomer_waits_until_the_pool_holds_all_its_tokens():
    """10 pages of 4 positions.  A (30 tokens, portions of 8) runs; B (20 tokens) would get its first portion
    at once, but not the pages for all its tokens beside what A will still ask for: admitted on the strength of
    that portion it would be preempted half-way and start again.  It waits; nothing is computed twice."""
    cache, s = make(num_pages=10, page_size=4, max_seqs=4, budget=16, chunk=8)
    s.add(req("A", 30, max_new=2))
    s.add(req("B", 20, max_new=2))
    s.add(req("C", 3, max_new=2))              # small enough to fit beside A, but behind B: first come first served
    computed = 0
    admitted_b_at = None
    steps = 0
    while s.has_work():
        plan, _ = run_step(s)
        computed += sum(p.n for p in plan)
        ids = [p.request.id for p in plan]
        if "B" in ids and admitted_b_at is None:
            admitted_b_at = steps
            a = next(r for r in s.finished + s.running if r.id == "A")
            assert a.remaining <= 1, "A had all its prompt pages before B came in"
        steps += 1
    assert s.num_preemptions == 0
    assert computed == sum(len(r.prompt) + len(r.output) - 1 for r in s.finished) == 30 + 20 + 3 + 3
    assert sorted(r.id for r in s.finished) == ["A", "B", "C"]
    assert admitted_b_at is not None and admitted_b_at >= 3


def test_a_request_larger_than_the_pool_does_not_hold_the_queue():
    cache, s = make(num_pages=6, page_size=4, max_seqs=4, budget=16, chunk=8)
    s.add(req("small", 5, max_new=2))
    s.add(req("big", 40, max_new=2))           # 40 tokens never fit into 24 positions
    s.add(req("next", 6, max_new=2))
    plan, _ = run_step(s)
    assert [p.request.id for p in plan] == ["small", "next"]
    big = next(r for r in s.finished if r.id == "big")
    assert big.finish_reason == "cache_full" and big.output == []
    while s.has_work():
        run_step(s)
    assert sorted(r.id for r in s.finished) == ["big", "next", "small"] and s.num_preemptions == 0
