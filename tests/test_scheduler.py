"""The scheduler's decisions, driven against the real cache bookkeeping with a
fake model (no GPU).  Cases follow the reference's scheduler tests
(crates/prelude-core/src/scheduler/tests.rs:51-1353): prefill then decode, the
token budget, the running limit, portions, mixed steps, admission by pages,
preemption, forced progress."""
import random

import pytest

from prelude_b200.cache.manager import CacheManager
from prelude_b200.engine.scheduler import CachePoolView, SamplingParams, Scheduler, SchedulerConfig
from prelude_b200.parts.registry import KvPagesNeed

EOS = (0,)


def make(num_pages=64, page=4, **kw):
    cache = CacheManager([KvPagesNeed(1, 16), KvPagesNeed(1, 16)], page, num_pages, 64, device=None)
    cfg = SchedulerConfig(page_size=page, **kw)
    return Scheduler(cfg, CachePoolView(cache)), cache


def drive(sched, cache, next_token=lambda seq: 1, max_steps=5000):
    """Run to completion; the cache grows exactly as the step function would grow it."""
    log = []
    while sched.has_work():
        items = sched.schedule()
        if not items:
            assert not sched.has_work()
            break
        assert len({it.seq.request_id for it in items}) == len(items)
        assert sum(it.n_tokens for it in items) <= sched.config.max_num_batched_tokens
        for it in items:
            rid = it.seq.request_id
            if not cache.has_request(rid):
                cache.add_request(rid)
            assert cache.tokens_of(rid) == it.start == it.seq.computed
            cache.grow(rid, it.start + it.n_tokens)          # the scheduler promised room: must not raise
            cache.trim(rid)
        cache.check()
        for it in items:
            sched.on_step_done(it, next_token(it.seq) if it.samples else None, EOS)
        log.append([(it.seq.request_id, it.start, it.n_tokens) for it in items])
        assert len(log) < max_steps
    return log


def P(n=4, **kw):
    return SamplingParams(max_new_tokens=n, temperature=0.0, **kw)


def test_prefill_then_decode_then_length():
    s, c = make()
    seq = s.add_request("a", [5] * 10, P(3), 128)
    log = drive(s, c)
    assert log == [[("a", 0, 10)], [("a", 10, 1)], [("a", 11, 1)]]
    assert seq.output == [1, 1, 1] and seq.finish_reason == "length"
    assert c.free_pages() == 64 and not c.requests


def test_budget_cuts_prompts_and_running_come_first():
    s, c = make(max_num_batched_tokens=8)
    s.add_request("a", [5] * 13, P(2), 128)
    s.add_request("b", [5] * 6, P(2), 128)
    log = drive(s, c)
    assert log[0] == [("a", 0, 8)]
    assert log[1] == [("a", 8, 5), ("b", 0, 3)]               # a finishes its prompt, b gets what is left
    assert log[2] == [("a", 13, 1), ("b", 3, 3)]              # a decoded token beside a prompt portion
    assert log[3] == [("b", 6, 1)]


def test_per_request_portion_cap():
    s, c = make(long_prefill_token_threshold=4)
    s.add_request("a", [5] * 10, P(1), 128)
    assert [step[0][2] for step in drive(s, c)] == [4, 4, 2]


def test_running_limit():
    s, c = make(max_running_requests=2)
    for i in range(4):
        s.add_request(i, [5] * 3, P(2), 128)
    log = drive(s, c)
    assert all(len(step) <= 2 for step in log)
    assert [r for r, _, _ in log[0]] == [0, 1]
    assert len(s.drain_finished()) == 4


def test_admission_waits_for_pages_and_reuses_them():
    s, c = make(num_pages=6, page=4, decode_reservation_cap=4)
    s.add_request("a", [5] * 12, P(4), 128)                   # 3 pages + 1 reserved
    s.add_request("b", [5] * 12, P(4), 128)                   # would need 4 more: only 2 left
    log = drive(s, c)
    first_b = next(i for i, step in enumerate(log) if any(r == "b" for r, _, _ in step))
    last_a = max(i for i, step in enumerate(log) if any(r == "a" for r, _, _ in step))
    assert first_b > last_a                                   # b waited until a gave its pages back
    assert s.stats["preemptions"] == 0


def test_decode_without_a_page_preempts_the_newest_and_rebuilds_its_cache():
    # two requests fit while they are short; both grow until the pool is full
    s, c = make(num_pages=6, page=4, decode_reservation_cap=0)
    a = s.add_request("a", [5] * 8, P(12), 128)
    b = s.add_request("b", [5] * 8, P(12), 128)
    log = drive(s, c)
    assert s.stats["preemptions"] >= 1
    assert b.preempt_count >= 1 and a.preempt_count == 0      # never the oldest
    assert len(a.output) == 12 and len(b.output) == 12
    # after the preemption b prefills prompt and generated tokens again, from position 0
    again = [e for step in log for e in step if e[0] == "b" and e[1] == 0]
    assert len(again) == 2 and again[1][2] > 8
    assert c.free_pages() == 6


def test_lone_request_that_cannot_fit_is_finished_with_cache_full():
    s, c = make(num_pages=2, page=4)
    seq = s.add_request("a", [5] * 20, P(4), 128)
    drive(s, c)
    assert seq.finish_reason == "cache_full" and seq.output == []
    s, c = make(num_pages=2, page=4)
    seq = s.add_request("a", [5] * 7, P(8), 128)              # fits, then outgrows the pool
    drive(s, c)
    assert seq.finish_reason == "cache_full" and len(seq.output) == 2
    assert c.free_pages() == 2


def test_forced_progress_when_the_reservation_does_not_fit():
    s, c = make(num_pages=4, page=4, decode_reservation_cap=4096)
    seq = s.add_request("a", [5] * 6, P(3), 128)              # 6 + min(3, cap) fits; make the reservation large instead
    seq.max_new_tokens = 1000
    seq.params.max_new_tokens = 1000
    log = drive(s, c, next_token=lambda q: 0 if len(q.output) == 2 else 1)
    assert s.stats["forced"] == 1 and log[0] == [("a", 0, 6)]
    assert seq.finish_reason == "eos"


def test_short_decode_tails_finish_before_new_prompts_are_admitted():
    s, c = make(decode_priority_max_remaining_tokens=4)
    s.add_request("a", [5] * 4, P(3), 128)
    drive_one = s.schedule()
    s.on_step_done(drive_one[0], 1, EOS)
    c.add_request("a"); c.grow("a", 4)
    s.add_request("b", [5] * 4, P(3), 128)
    step = s.schedule()
    assert [it.seq.request_id for it in step] == ["a"]       # a has 2 tokens left: b waits


def test_stop_reasons_and_order():
    s, c = make()
    a = s.add_request("a", [5] * 3, P(10), 128)
    b = s.add_request("b", [5] * 3, P(10, stop_token_ids=(7,)), 128)
    d = s.add_request("d", [5] * 3, P(10, ignore_eos=True), 128)
    toks = {"a": [3, 0, 9], "b": [3, 7, 9], "d": [0, 0] + [2] * 20}
    drive(s, c, next_token=lambda q: toks[q.request_id][len(q.output)])
    assert (a.finish_reason, a.output) == ("eos", [3, 0])
    assert (b.finish_reason, b.output) == ("stop", [3, 7])
    assert d.finish_reason == "length" and len(d.output) == 10


def test_max_new_is_clamped_to_the_context():
    s, c = make()
    seq = s.add_request("a", [5] * 10, P(100), 16)
    drive(s, c)
    assert len(seq.output) == 6
    with pytest.raises(ValueError):
        s.add_request("b", [5] * 16, P(1), 16)
    with pytest.raises(ValueError):
        s.add_request("c", [], P(1), 16)


def test_abort_gives_everything_back():
    s, c = make()
    s.add_request("a", [5] * 9, P(5), 128)
    s.add_request("b", [5] * 9, P(5), 128)
    items = s.schedule()
    for it in items:
        c.add_request(it.seq.request_id); c.grow(it.seq.request_id, it.n_tokens)
        s.on_step_done(it, 1, EOS)
    assert s.abort("a") and not s.abort("zzz")
    assert not c.has_request("a") and c.has_request("b")
    drive(s, c)
    reasons = {q.request_id: q.finish_reason for q in s.drain_finished()}
    assert reasons == {"a": "abort", "b": "length"}
    assert c.free_pages() == 64


def test_max_total_tokens_preempts_the_newest():
    s, c = make(max_total_tokens=24)
    a = s.add_request("a", [5] * 10, P(6), 128)
    b = s.add_request("b", [5] * 10, P(6), 128)
    drive(s, c)
    assert len(a.output) == 6 and len(b.output) == 6
    assert a.preempt_count == 0


@pytest.mark.parametrize("seed", range(8))
def test_random_load_always_finishes_and_keeps_the_books(seed):
    rng = random.Random(seed)
    pages, page = rng.choice([(12, 4), (20, 8), (40, 2)])
    s, c = make(num_pages=pages, page=page, max_num_batched_tokens=rng.choice([5, 16, 64]),
                long_prefill_token_threshold=rng.choice([0, 3, 7]), max_running_requests=rng.choice([2, 4, 8]),
                decode_reservation_cap=rng.choice([0, 4, 4096]))
    seqs = []
    for i in range(12):
        n = rng.randint(1, 30)
        seqs.append(s.add_request(i, [rng.randint(1, 50) for _ in range(n)], P(rng.randint(1, 12)), 64))
    drive(s, c, next_token=lambda q: rng.choice([1, 1, 1, 1, 0]))
    for q in seqs:
        assert q.finish_reason in ("eos", "length", "cache_full")
        if q.finish_reason == "length":
            assert len(q.output) == q.max_new_tokens
        if q.finish_reason == "cache_full":
            assert q.total_len + 1 > pages * page or len(q.prompt) > pages * page
    assert c.free_pages() == pages and not c.requests
    c.check()
