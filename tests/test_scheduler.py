"""The scheduler's decisions, driven on the host with the real cache manager and a
stand-in for the model that appends the pages the scheduler planned (no GPU)."""
import random

import pytest

from vllm_lite_b200.cache import CacheLayout, CacheManager, PagedKV
from vllm_lite_b200.cache.native import NativeCacheManager

BACKEND = {"cls": CacheManager, "native_policy": None}


@pytest.fixture(autouse=True, params=["python", "native", "native cache, python policy"])
def cache_backend(request):
    """Every test runs with the Python cache manager and policy, with the C++ core for both, and
    with the C++ cache core under the Python policy."""
    BACKEND["cls"] = CacheManager if request.param == "python" else NativeCacheManager
    BACKEND["native_policy"] = {"python": False, "native": True}.get(request.param, False)
    yield
from vllm_lite_b200.engine.scheduler import AdmissionError, Scheduler, SchedulerConfig
from vllm_lite_b200.sampling import SamplingParams


def make(num_pages=64, page_size=4, max_requests=8, **cfg):
    lay = CacheLayout.from_needs([PagedKV(2, 16)], [None])
    cache = BACKEND["cls"](lay, page_size, num_pages, max_requests)
    return cache, Scheduler(cache, SchedulerConfig(**cfg), native=BACKEND["native_policy"])


def run_step(cache, sched, token_of=lambda seq: 7):
    """What the engine does around a step: take the pages, 'sample', update."""
    plan = sched.schedule()
    for e in plan.entries:
        if e.seq.seq_id not in cache.requests:
            cache.admit(e.seq.seq_id)
        assert cache.requests[e.seq.seq_id].num_tokens == e.start
        if e.start == e.seq.num_computed:              # the scheduler's own count of pages is the cache manager's
            assert sched._pages_needed(e.seq, e.count) == cache.pages_needed(e.seq.seq_id, e.count)
        cache.append(e.seq.seq_id, e.count)            # must never raise: the scheduler counted the pages
    sampled = [token_of(e.seq) if e.samples else None for e in plan.entries]
    done = sched.update(plan, sampled)
    cache.check_invariants()
    return plan, done


def test_first_come_first_served_under_a_token_budget():
    cache, s = make(max_num_batched_tokens=10, prefill_chunk_size=6)
    a = s.add_request(range(9), 3)
    b = s.add_request(range(4), 2)
    plan, _ = run_step(cache, s)
    # nobody decodes yet: prefill_chunk_size does not bound the portions, the token budget does
    assert [(e.seq.seq_id, e.start, e.count, e.samples) for e in plan.entries] == [(a.seq_id, 0, 9, True), (b.seq_id, 0, 1, False)]
    assert plan.num_tokens <= 10
    plan, _ = run_step(cache, s)
    # a decodes (one token, first), b finishes its prompt beside it
    assert [(e.seq.seq_id, e.start, e.count, e.samples) for e in plan.entries] == [(a.seq_id, 9, 1, True), (b.seq_id, 1, 3, True)]
    plan, _ = run_step(cache, s)
    assert [(e.seq.seq_id, e.count) for e in plan.entries] == [(a.seq_id, 1), (b.seq_id, 1)]
    assert b.status == "finished" and b.finish_reason == "length" and b.generated == [7, 7]
    assert a.status == "finished" and len(a.generated) == 3
    assert cache.free_pages() == [64] and not s.has_work()
    assert s.stats["prefill_tokens"] == 13 and s.stats["decode_tokens"] == 3 and s.stats["finished"] == 2


def test_prefill_chunk_size_bounds_portions_only_beside_decoding_requests():
    cache, s = make(max_num_batched_tokens=32, prefill_chunk_size=6)
    a = s.add_request(range(5), 8)
    run_step(cache, s)                                   # a's prompt; from now on a decodes
    b = s.add_request(range(20), 2)
    plan, _ = run_step(cache, s)
    assert [(e.seq.seq_id, e.count) for e in plan.entries] == [(a.seq_id, 1), (b.seq_id, 6)]   # a's token must not wait long
    plan, _ = run_step(cache, s)
    assert [(e.seq.seq_id, e.count) for e in plan.entries] == [(a.seq_id, 1), (b.seq_id, 6)]
    s.cancel(a.seq_id)
    plan, _ = run_step(cache, s)
    assert [(e.seq.seq_id, e.start, e.count) for e in plan.entries] == [(b.seq_id, 12, 8)]     # alone again: all that is left
    c = s.add_request(range(40), 2)                      # and a prompt beyond the budget is cut by the budget
    plan, _ = run_step(cache, s)
    assert [(e.seq.seq_id, e.count) for e in plan.entries] == [(b.seq_id, 1), (c.seq_id, 6)]
    assert b.status == "finished"
    plan, _ = run_step(cache, s)
    assert [(e.seq.seq_id, e.start, e.count) for e in plan.entries] == [(c.seq_id, 6, 32)]     # 34 left, 32 fit the budget


def test_n_tokens_take_one_prompt_step_and_n_minus_one_decode_steps():
    cache, s = make()
    seq = s.add_request([1, 2, 3], 5)
    steps = 0
    while s.has_work():
        run_step(cache, s)
        steps += 1
    assert steps == 5 and len(seq.generated) == 5 and seq.num_computed == 3 + 4


def test_max_num_seqs_and_head_of_line_blocking():
    cache, s = make(num_pages=8, max_num_seqs=2)
    a = s.add_request(range(8), 4)          # 2 pages now
    b = s.add_request(range(20), 4)         # 5 pages
    c = s.add_request(range(2), 4)          # would fit, but waits behind b
    d = s.add_request(range(2), 4)
    plan, _ = run_step(cache, s)
    assert [e.seq.seq_id for e in plan.entries] == [a.seq_id, b.seq_id]
    assert [q.seq_id for q in s.waiting] == [c.seq_id, d.seq_id]          # max_num_seqs = 2
    while a.status != "finished":
        plan, _ = run_step(cache, s)
    assert c.status == "waiting"
    run_step(cache, s)                       # a's place is free now: c is admitted, d still waits
    assert c.status == "running" and d.status == "waiting"


def test_requests_that_can_never_fit_are_rejected_at_admission():
    cache, s = make(num_pages=4, page_size=4, max_model_len=64)
    with pytest.raises(AdmissionError):
        s.add_request([], 4)
    with pytest.raises(AdmissionError):
        s.add_request(range(10), 8)            # 18 tokens > 16 slots in the pool
    with pytest.raises(AdmissionError):
        s.add_request(range(60), 8)            # beyond max_model_len
    with pytest.raises(AdmissionError):
        s.add_request(range(3), 0)
    s.add_request(range(10), 6)


def test_when_pages_run_out_the_newest_request_is_recomputed():
    cache, s = make(num_pages=6, page_size=4)
    a = s.add_request(range(8), 12)            # grows to 20 tokens = 5 pages
    b = s.add_request(range(7), 10)            # grows to 17 tokens
    preempted = []
    tokens = {a.seq_id: iter(range(100, 200)), b.seq_id: iter(range(200, 300))}
    for _ in range(200):
        if not s.has_work():
            break
        plan, _ = run_step(cache, s, token_of=lambda seq: next(tokens[seq.seq_id]))
        preempted += [p.seq_id for p in plan.preempted]
    assert not s.has_work()
    assert preempted and set(preempted) == {b.seq_id}           # the older request is never the victim
    assert a.preemptions == 0 and b.preemptions >= 1
    # the generated tokens survive pre-emption and nothing is sampled twice
    assert a.generated == list(range(100, 112)) and b.generated == list(range(200, 210))
    assert cache.free_pages() == [6] and s.stats["preemptions"] == len(preempted)


def test_stop_sequences_and_cancel():
    cache, s = make()
    a = s.add_request([1], 50, SamplingParams(stop_token_sequences=[[5, 6]]))
    b = s.add_request([2], 50)
    feed = iter([4, 0, 5, 0, 6, 0, 9, 0])
    run_step(cache, s, token_of=lambda seq: next(feed))
    assert s.cancel(b.seq_id) and b.finish_reason == "cancelled" and not s.cancel(b.seq_id)
    feed = iter([5, 6, 9])
    while s.has_work():
        run_step(cache, s, token_of=lambda seq: next(feed))
    assert a.finish_reason == "stop" and a.generated == [4, 5, 6]
    assert cache.free_pages() == [64]


@pytest.mark.parametrize("seed", range(6))
def test_random_traffic_never_leaks_or_exceeds_limits(seed):
    rng = random.Random(seed)
    cache, s = make(num_pages=30, page_size=4, max_requests=6, max_num_seqs=6, max_num_batched_tokens=24, prefill_chunk_size=9)
    seqs = []
    for step in range(400):
        if rng.random() < 0.3 and len(seqs) < 40:
            seqs.append(s.add_request([rng.randrange(50) for _ in range(rng.randint(1, 40))], rng.randint(1, 30)))
        if s.has_work():
            plan, _ = run_step(cache, s)
            assert plan.num_tokens <= 24 and len(s.running) <= 6
            ids = [e.seq.seq_id for e in plan.entries]
            assert len(ids) == len(set(ids))
    while s.has_work():
        run_step(cache, s)
    assert all(q.status == "finished" and len(q.generated) == q.max_tokens for q in seqs)
    assert cache.free_pages() == [30] and cache.slots.free_count == 6


@pytest.mark.parametrize("seed", range(5))
def test_the_native_policy_decides_as_the_python_policy(seed):
    """Two engines' worth of host state fed the same traffic, one deciding in Python and one in the
    C++ core: the same entries, the same victims, step by step, through admissions, portions,
    pre-emptions and a pool with a window."""
    rng = random.Random(100 + seed)
    lay = CacheLayout.from_needs([PagedKV(2, 16), PagedKV(1, 8, window=11)], [None, None])
    cfg = dict(max_num_seqs=5, max_num_batched_tokens=20, prefill_chunk_size=7)
    pair = []
    for native in (False, True):
        cache = NativeCacheManager(lay, 4, [26, 40], 5)
        pair.append((cache, Scheduler(cache, SchedulerConfig(**cfg), native=native)))
    assert pair[0][1].native is False and pair[1][1].native is True
    added = 0
    for step in range(300):
        if rng.random() < 0.35 and added < 30:
            prompt, mt = [rng.randrange(50) for _ in range(rng.randint(1, 30))], rng.randint(1, 25)
            for _, s in pair:
                s.add_request(prompt, mt)
            added += 1
        plans = []
        for cache, s in pair:
            if not s.has_work():
                plans.append(None)
                continue
            plan = s.schedule()
            for e in plan.entries:
                if e.seq.seq_id not in cache.requests:
                    cache.admit(e.seq.seq_id)
                cache.append(e.seq.seq_id, e.count)
                cache.release_behind_window(e.seq.seq_id)
            s.update(plan, [7 if e.samples else None for e in plan.entries])
            cache.check_invariants()
            plans.append(([(e.seq.seq_id, e.start, e.count, e.samples) for e in plan.entries],
                          [v.seq_id for v in plan.preempted]))
        assert plans[0] == plans[1], (step, plans)
    assert pair[0][1].stats == pair[1][1].stats and pair[0][1].stats["preemptions"] > 0
