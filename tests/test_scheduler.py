"""The scheduler's decisions (CPU): admission, portions under a token budget, decode first,
finishing and freeing, and what happens when pages run out."""
import random
import zlib

import pytest

from infinicore_infer_b200.cache import CacheManager, PagedKV
from infinicore_infer_b200.engine.scheduler import FINISHED, RUNNING, WAITING, Request, Scheduler


def fake_token(seq, vocab=1000):
    """A stand-in for the model: the next token is a function of the whole sequence so far."""
    return zlib.crc32(bytes(str(list(seq)), "ascii")) % vocab


class FakeEngine:
    """Does to the cache manager what Engine.step does, and 'samples' with fake_token."""

    def __init__(self, cache):
        self.cache = cache
        self.steps = []

    def run(self, plan):
        wants = {}
        for s in plan:
            r = s.request
            if not self.cache.is_live(r.id):
                self.cache.admit(r.id)
            assert self.cache.length(r.id) == r.computed
            wants[r.id] = r.computed + len(s.tokens)
        assert self.cache.can_reserve(wants), "the scheduler planned a step that does not fit"
        out = []
        for s in plan:
            r = s.request
            self.cache.reserve(r.id, wants[r.id])
            self.cache.commit(r.id, wants[r.id])
            assert s.tokens == r.tokens[r.computed:r.computed + len(s.tokens)]
            out.append(fake_token(r.tokens[:r.computed + len(s.tokens)]) if s.samples else None)
        self.steps.append([(s.request.id, len(s.tokens), s.samples) for s in plan])
        self.cache.check_invariants()
        return out


def make(num_pages=64, page=4, max_requests=8, max_positions=256, **kw):
    cache = CacheManager([PagedKV(2, 16), PagedKV(2, 16)], num_pages, page, max_requests, max_positions, device=None)
    return cache, Scheduler(cache, **kw), FakeEngine(cache)


def drive(sched, eng, limit=10000):
    n = 0
    while sched.has_work():
        plan = sched.schedule()
        sched.complete(plan, eng.run(plan))
        n += 1
        assert n < limit, "the scheduler does not terminate"
    return n


def expected_output(prompt, n, eos=()):
    seq, out = list(prompt), []
    for _ in range(n):
        t = fake_token(seq)
        out.append(t); seq.append(t)
        if t in eos:
            break
    return out


def test_a_prompt_is_cut_into_portions_under_the_budget():
    cache, sched, eng = make(max_batch=4, max_tokens_per_step=10, chunk_size=7)
    r = Request("a", list(range(23)), max_new_tokens=3)
    sched.add(r)
    drive(sched, eng)
    sizes = [s[0][1] for s in eng.steps]
    assert sizes == [7, 7, 7, 2, 1, 1]                 # portions of the chunk size, the rest, then decoding
    assert [s[0][2] for s in eng.steps] == [False, False, False, True, True, True]
    assert r.generated == expected_output(range(23), 3) and r.finish_reason == "length"
    assert not cache.is_live("a") and cache.groups[0].pool.in_use == 0 and cache.slots.available == 8


def test_decoding_requests_come_first_and_portions_fill_the_rest_of_the_budget():
    cache, sched, eng = make(max_batch=4, max_tokens_per_step=12, chunk_size=8)
    a = Request("a", list(range(5)), max_new_tokens=6)
    sched.add(a)
    plan = sched.schedule(); sched.complete(plan, eng.run(plan))       # a's prompt; a now decodes
    b = Request("b", list(range(100, 130)), max_new_tokens=2)
    c = Request("c", list(range(200, 209)), max_new_tokens=2)
    sched.add(b); sched.add(c)
    plan = sched.schedule()
    assert [(s.request.id, len(s.tokens)) for s in plan] == [("a", 1), ("b", 8), ("c", 3)]
    assert sum(len(s.tokens) for s in plan) == 12
    sched.complete(plan, eng.run(plan))
    plan = sched.schedule()
    assert [(s.request.id, len(s.tokens), s.samples) for s in plan] == [("a", 1, True), ("b", 8, False), ("c", 3, False)]
    sched.complete(plan, eng.run(plan))
    drive(sched, eng)
    for r in (a, b, c):
        assert r.generated == expected_output(r.prompt, r.max_new_tokens)
    assert all(sum(n for _, n, _ in step) <= 12 for step in eng.steps)


def test_finish_reasons_and_immediate_freeing():
    cache, sched, eng = make()
    prompt = [3, 1, 4]
    eos = expected_output(prompt, 3)[2]
    a = Request("a", prompt, max_new_tokens=10, eos_token_ids=(eos,))
    b = Request("b", [9, 9], max_new_tokens=2)
    sched.add(a); sched.add(b)
    drive(sched, eng)
    assert a.finish_reason == "stop" and a.generated == expected_output(prompt, 3) and a.generated[-1] == eos
    assert b.finish_reason == "length" and len(b.generated) == 2
    assert a.status == FINISHED and cache.slots.available == 8
    assert all(g.pool.in_use == 0 for g in cache.groups)


def test_context_limit_finishes_with_length():
    cache, sched, eng = make(max_positions=12)
    a = Request("a", list(range(9)), max_new_tokens=50)
    sched.add(a)
    drive(sched, eng)
    assert a.finish_reason == "length" and a.computed <= 12
    assert len(a.prompt) + len(a.generated) == 13      # the 13th token was sampled but cannot be fed
    too_long = Request("b", list(range(13)), max_new_tokens=1)
    sched.add(too_long)
    drive(sched, eng)
    assert too_long.finish_reason == "length" and too_long.generated == []


def test_max_batch_and_slots_bound_the_running_set():
    cache, sched, eng = make(max_requests=3, max_batch=2, max_tokens_per_step=64, chunk_size=64)
    reqs = [Request(i, [i, i + 1, i + 2], max_new_tokens=4) for i in range(5)]
    for r in reqs:
        sched.add(r)
    while sched.has_work():
        plan = sched.schedule()
        assert len(sched.running) <= 2 and len(plan) <= 2
        sched.complete(plan, eng.run(plan))
    assert [r.generated for r in reqs] == [expected_output(r.prompt, 4) for r in reqs]
    # requests were served in arrival order
    first_seen = []
    for step in eng.steps:
        for rid, _, _ in step:
            if rid not in first_seen:
                first_seen.append(rid)
    assert first_seen == [0, 1, 2, 3, 4]


def test_admission_waits_until_the_first_portion_fits():
    cache, sched, eng = make(num_pages=6, page=4, max_tokens_per_step=64, chunk_size=16)
    a = Request("a", list(range(16)), max_new_tokens=30)       # 4 pages, then one more every 4 tokens
    b = Request("b", list(range(50, 62)), max_new_tokens=2)    # 3 pages
    sched.add(a); sched.add(b)
    plan = sched.schedule()
    assert [s.request.id for s in plan] == ["a"] and b.status == WAITING
    sched.complete(plan, eng.run(plan))
    drive(sched, eng)
    assert a.generated == expected_output(a.prompt, len(a.generated)) and b.generated == expected_output(b.prompt, 2)


def test_when_pages_run_out_the_youngest_is_preempted_and_recomputed():
    cache, sched, eng = make(num_pages=10, page=4, max_tokens_per_step=64, chunk_size=64)
    a = Request("a", list(range(10)), max_new_tokens=20)
    b = Request("b", list(range(100, 110)), max_new_tokens=20)
    sched.add(a); sched.add(b)
    drive(sched, eng)
    # both need 8 pages at the end (30 tokens), the pool has 10: they cannot both finish side by side
    assert sched.counters["preemptions"] >= 1 and b.preemptions >= 1 and a.preemptions == 0
    assert a.generated == expected_output(a.prompt, 20) and b.generated == expected_output(b.prompt, 20)
    # after the preemption b came back with prompt + generated as one prompt, cut into portions again
    restarts = [step for step in eng.steps if any(rid == "b" and n > 1 for rid, n, _ in step)]
    assert len(restarts) >= 2
    assert all(g.pool.in_use == 0 for g in cache.groups)


def test_a_request_that_cannot_fit_alone_finishes_with_length():
    cache, sched, eng = make(num_pages=3, page=4, max_tokens_per_step=64, chunk_size=64)
    big = Request("big", list(range(20)), max_new_tokens=5)      # 5 pages > 3
    ok = Request("ok", list(range(6)), max_new_tokens=50)        # grows until the pool is full
    sched.add(big); sched.add(ok)
    drive(sched, eng)
    assert big.finish_reason == "length" and big.generated == []
    assert ok.finish_reason == "length" and 0 < len(ok.generated) < 50
    assert len(ok.prompt) + len(ok.generated) - 1 <= 12          # it stopped when a fourth page was needed
    assert ok.generated == expected_output(ok.prompt, len(ok.generated))
    assert all(g.pool.in_use == 0 for g in cache.groups)


def test_a_portion_shrinks_to_the_pages_that_are_free():
    cache, sched, eng = make(num_pages=8, page=4, max_tokens_per_step=64, chunk_size=64)
    a = Request("a", list(range(12)), max_new_tokens=40)
    sched.add(a)
    plan = sched.schedule(); sched.complete(plan, eng.run(plan))
    b = Request("b", list(range(100, 140)), max_new_tokens=1)    # 10 pages: never fits beside a, fits alone? no: 8 pages
    c = Request("c", list(range(200, 216)), max_new_tokens=1)    # 4 pages
    sched.add(c)
    plan = sched.schedule()
    assert [(s.request.id, len(s.tokens)) for s in plan] == [("a", 1), ("c", 16)]
    sched.complete(plan, eng.run(plan))
    drive(sched, eng)
    assert c.generated == expected_output(c.prompt, 1)
    sched.add(b)
    drive(sched, eng)
    assert b.finish_reason == "length" and b.generated == []


def test_cancel_frees_at_once():
    cache, sched, eng = make()
    a = Request("a", list(range(9)), max_new_tokens=50)
    sched.add(a)
    plan = sched.schedule(); sched.complete(plan, eng.run(plan))
    assert cache.is_live("a")
    assert sched.cancel("a") and a.finish_reason == "cancel" and not cache.is_live("a")
    assert not sched.cancel("a") and not sched.has_work()


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_give_the_same_tokens_as_an_unconstrained_run(seed):
    rng = random.Random(seed)
    cache, sched, eng = make(num_pages=rng.randint(14, 30), page=rng.choice([2, 4, 8]), max_requests=4,
                             max_positions=200, max_batch=4, max_tokens_per_step=rng.choice([8, 16, 40]),
                             chunk_size=rng.choice([3, 9, 32]))
    reqs = []
    pending = [Request(i, [rng.randrange(1000) for _ in range(rng.randint(1, 40))],
                       max_new_tokens=rng.randint(1, 25)) for i in range(12)]
    steps = 0
    while pending or sched.has_work():
        if pending and rng.random() < 0.4:
            r = pending.pop(0); reqs.append(r); sched.add(r)
        if sched.has_work():
            plan = sched.schedule()
            assert sum(len(s.tokens) for s in plan) <= sched.max_tokens_per_step
            assert len({s.request.id for s in plan}) == len(plan)
            # decoding rows first
            kinds = [s.request.decoding for s in plan]
            assert kinds == sorted(kinds, reverse=True)
            sched.complete(plan, eng.run(plan))
        steps += 1
        assert steps < 5000
    for r in reqs:
        assert r.status == FINISHED
        if r.finish_reason == "length" and len(r.generated) < r.max_new_tokens:
            continue                                   # could not fit alone
        assert r.generated == expected_output(r.prompt, r.max_new_tokens), (r.id, r.preemptions)
    assert all(g.pool.in_use == 0 for g in cache.groups) and cache.slots.available == 4
