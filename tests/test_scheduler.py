"""The scheduler's decisions (no GPU, no torch).  The first group mirrors the reference's
scheduler tests (tests/test_scheduler.py:121-243); the second covers what the reference has
not: token budget, prompt portions, mixed steps, preemption half-way through a prompt."""

from __future__ import annotations

import pytest

from mini_gpt_inference_b200.cache import CacheManager, PagedKVSpec
from mini_gpt_inference_b200.config import SamplingParams
from mini_gpt_inference_b200.engine.request import Request, SequenceState, SequenceStatus
from mini_gpt_inference_b200.engine.scheduler import Scheduler


def make(num_pages=8, page_tokens=4, max_batch=4, budget=64, chunk=None, policy="prefill_priority"):
    cache = CacheManager([PagedKVSpec(2, 8)], page_tokens, num_pages, max_batch)
    return cache, Scheduler(cache, max_batch, budget, chunk, policy)


def seq(rid, prompt_len, max_tokens=8):
    return SequenceState(Request(rid, list(range(1, prompt_len + 1)), SamplingParams(max_tokens=max_tokens)))


def run_step(sched, chunks, token=7):
    """What the engine does after a step: count the tokens in, append the sampled ones."""
    for c in chunks:
        c.seq.num_computed_tokens += c.count
    for c in chunks:
        if c.samples:
            c.seq.output_token_ids.append(token)


def test_admits_up_to_max_batch_size_in_fifo_order():
    cache, s = make(num_pages=32, max_batch=2)
    seqs = [seq(f"r{i}", 3) for i in range(3)]
    for q in seqs:
        s.add_request(q)
    chunks = s.schedule()
    assert [c.seq.request_id for c in chunks] == ["r0", "r1"]
    assert all(c.samples and c.start == 0 and c.count == 3 for c in chunks)
    assert seqs[2].status == SequenceStatus.WAITING and len(s.running) == 2


def test_decodes_when_nothing_to_admit_and_prompts_come_first():
    cache, s = make(num_pages=32, budget=16)
    a = seq("a", 3)
    s.add_request(a)
    run_step(s, s.schedule())
    chunks = s.schedule()
    assert [(c.seq.request_id, c.start, c.count, c.samples) for c in chunks] == [("a", 3, 1, True)]
    run_step(s, chunks)
    b = seq("b", 5)
    s.add_request(b)
    chunks = s.schedule()                                  # one mixed step: a decodes, b's prompt
    assert {(c.seq.request_id, c.count) for c in chunks} == {("a", 1), ("b", 5)}


def test_head_of_line_request_blocks_the_queue():
    cache, s = make(num_pages=4, page_tokens=4)
    s.add_request(seq("big", 13, max_tokens=1))
    s.add_request(seq("small", 2, max_tokens=1))
    run_step(s, s.schedule())                              # big takes all 4 pages
    assert [q.request_id for q in s.running] == ["big"] and cache.num_free_pages() == 0
    s.add_request(seq("late", 2, max_tokens=1))
    chunks = s.schedule()
    assert [c.seq.request_id for c in chunks] == ["big"]   # nobody jumps the queue
    assert [q.request_id for q in s.waiting] == ["small", "late"]


def test_finish_frees_pages_in_the_same_step_and_cancel_works():
    cache, s = make()
    a, b = seq("a", 6), seq("b", 2)
    s.add_request(a)
    s.add_request(b)
    run_step(s, s.schedule())
    assert cache.num_free_pages() == 8 - 2 - 1
    s.finish(a, "length")
    assert cache.num_free_pages() == 7 and a.finish_reason == "length" and a not in s.running
    assert s.cancel_by_id("b") and b.finish_reason == "cancelled" and cache.num_free_pages() == 8
    c = seq("c", 2)
    s.add_request(c)
    assert s.cancel_by_id("c") and not s.waiting and c.is_finished()
    assert not s.cancel_by_id("nobody")
    cache.check()


def test_preempts_newest_and_puts_it_at_the_front():
    cache, s = make(num_pages=4, page_tokens=2, max_batch=3)
    a, b, c = seq("a", 2, 4), seq("b", 2, 4), seq("c", 2, 4)
    for q in (a, b, c):
        s.add_request(q)
    run_step(s, s.schedule())                              # 3 pages out, 1 free
    s.add_request(seq("d", 2, 4))
    chunks = s.schedule()                                  # a takes the last page; b needs one: c goes
    assert s.num_preemptions >= 1
    assert c.status == SequenceStatus.WAITING and c.num_computed_tokens == 0
    assert s.waiting[0] is c                               # ahead of d
    assert [x.seq.request_id for x in chunks] == ["a", "b"]
    assert c.output_token_ids == [7]                       # what it generated is kept and recomputed
    cache.check()


def test_lone_request_that_cannot_grow_preempts_itself():
    cache, s = make(num_pages=3, page_tokens=2, max_batch=2)
    a = seq("a", 4, max_tokens=2)
    s.add_request(a)
    run_step(s, s.schedule())                              # 2 pages
    cache.admit("someone-else")                            # a holder outside the scheduler
    assert cache.reserve("someone-else", 2)                # takes the last page
    chunks = s.schedule()                                  # a needs a third page; nobody to preempt
    assert chunks == [] and a.status == SequenceStatus.WAITING and s.num_preemptions == 1
    assert a.num_computed_tokens == 0 and cache.num_free_pages() == 2


def test_request_that_can_never_fit_is_refused_when_added():
    cache, s = make(num_pages=2, page_tokens=4)
    s.add_request(seq("just", 8, max_tokens=1))            # 8 tokens in the cache at most
    with pytest.raises(ValueError, match="never fit"):
        s.add_request(seq("huge", 8, max_tokens=2))


def test_token_budget_cuts_prompts_into_portions():
    cache, s = make(num_pages=64, budget=10, chunk=6)
    a, b = seq("a", 14), seq("b", 3)
    s.add_request(a)
    s.add_request(b)
    c1 = s.schedule()
    assert [(c.seq.request_id, c.start, c.count, c.samples) for c in c1] == [
        ("a", 0, 6, False), ("b", 0, 3, True)]
    run_step(s, c1)
    c2 = s.schedule()                                      # a's prompt goes on first, then b decodes
    assert [(c.seq.request_id, c.start, c.count, c.samples) for c in c2] == [
        ("a", 6, 6, False), ("b", 3, 1, True)]
    run_step(s, c2)
    c3 = s.schedule()
    assert [(c.seq.request_id, c.start, c.count, c.samples) for c in c3] == [
        ("a", 12, 2, True), ("b", 4, 1, True)]
    assert sum(c.count for c in c1) <= 10


def test_budget_exhausted_by_prompts_leaves_decodes_waiting_and_decode_priority_reverses_it():
    for policy, first in (("prefill_priority", "p"), ("decode_priority", "d")):
        cache, s = make(num_pages=64, budget=4, chunk=4, policy=policy)
        d = seq("d", 2)
        s.add_request(d)
        run_step(s, s.schedule())
        p = seq("p", 12)
        s.add_request(p)
        run_step(s, s.schedule())                          # d decodes (1) + p's first 3
        chunks = s.schedule()
        assert chunks[0].seq.request_id == first
        assert sum(c.count for c in chunks) <= 4


def test_preemption_half_way_through_a_prompt_restarts_it():
    cache, s = make(num_pages=5, page_tokens=2, max_batch=2, budget=4, chunk=4)
    old = seq("old", 3, max_tokens=6)
    s.add_request(old)
    run_step(s, s.schedule())                              # old: 2 pages
    young = seq("young", 7, max_tokens=1)
    s.add_request(young)
    run_step(s, s.schedule())                              # old decodes (same page), young 3 of 7 -> 2 pages
    assert young.num_computed_tokens == 3 and not young.output_token_ids
    # young's portion shrinks to the one free page and takes it; then old needs a page to
    # decode, and the newest other request, half-way through its prompt, gives way
    chunks = s.schedule()
    assert s.num_preemptions == 1
    assert young.num_computed_tokens == 0 and s.waiting[0] is young
    assert young.status == SequenceStatus.WAITING
    assert [c.seq.request_id for c in chunks] == ["old"]
    cache.check()
    # young is recomputed from its first token once old is done
    s.finish(old, "length")
    again = s.schedule()
    assert [(c.seq.request_id, c.start) for c in again] == [("young", 0)]


def test_prompt_portion_shrinks_to_free_pages_instead_of_preempting():
    cache, s = make(num_pages=4, page_tokens=2, max_batch=2, budget=8, chunk=4)
    cache.admit("holder")                                  # a holder outside the scheduler
    assert cache.reserve("holder", 2)                      # keeps one page
    with pytest.raises(ValueError, match="never fit"):
        s.add_request(seq("toolong", 9, 1))
    a = seq("a", 7, max_tokens=1)
    s.add_request(a)
    c1 = s.schedule()
    assert [(c.start, c.count, c.samples) for c in c1] == [(0, 4, False)]
    run_step(s, c1)
    c2 = s.schedule()                                      # wants 3 more, one page free: 2 tokens
    assert [(c.start, c.count, c.samples) for c in c2] == [(4, 2, False)]
    run_step(s, c2)
    cache.release("holder")
    c3 = s.schedule()
    assert [(c.start, c.count, c.samples) for c in c3] == [(6, 1, True)]
    assert s.num_preemptions == 0
    cache.check()


def test_stuck_requests_resolve_by_newest_giving_way():
    cache, s = make(num_pages=4, page_tokens=2, max_batch=2, budget=4, chunk=2)
    a, b = seq("a", 6, 1), seq("b", 6, 1)
    s.add_request(a)
    s.add_request(b)
    run_step(s, s.schedule())                              # a: 2 tokens, b: 2 tokens
    run_step(s, s.schedule())                              # a: 4, b: 4 -> pool empty, both need more
    chunks = s.schedule()                                  # both stuck: b gives way, a moves
    assert s.num_preemptions == 1 and b.status == SequenceStatus.WAITING
    assert [(c.seq.request_id, c.start, c.count) for c in chunks] == [("a", 4, 2)]
    cache.check()


def test_everything_is_given_back_after_a_busy_run():
    import random

    rng = random.Random(1)
    cache, s = make(num_pages=10, page_tokens=2, max_batch=4, budget=6, chunk=3)
    seqs = [seq(f"r{i}", rng.randint(1, 7), max_tokens=rng.randint(1, 6)) for i in range(25)]
    pending = list(seqs)
    steps = 0
    while pending or s.has_work():
        if pending and rng.random() < 0.5:
            s.add_request(pending.pop(0))
        chunks = s.schedule()
        assert sum(c.count for c in chunks) <= 6 and len(s.running) <= 4
        run_step(s, chunks)
        for c in chunks:
            if c.samples and len(c.seq.output_token_ids) >= c.seq.request.sampling_params.max_tokens:
                s.finish(c.seq, "length")
        cache.check()
        steps += 1
        assert steps < 5000
    assert cache.num_free_pages() == 10 and cache.slots.num_free == 4
    assert all(q.is_finished() for q in seqs) and s.num_preemptions > 0
    assert all(len(q.output_token_ids) == q.request.sampling_params.max_tokens for q in seqs)


def test_steady_decode_schedule_looks_at_counts_only():
    cache, s = make(num_pages=8, page_tokens=2, max_batch=3, budget=16)
    a, b = seq("a", 3, max_tokens=3), seq("b", 2, max_tokens=8)
    s.add_request(a)
    s.add_request(b)
    assert s.schedule_steady_decode() is None               # somebody waits: general path
    run_step(s, s.schedule())                               # prompts in, first tokens sampled
    rows = s.schedule_steady_decode()
    assert [q.request_id for q in rows] == ["a", "b"]
    free = cache.num_free_pages()
    # the engine launches the step and counts the new tokens as in flight, values unknown
    for q in rows:
        q.num_computed_tokens += 1
        q.num_inflight += 1
    for q in rows:                                          # ... their ids arrive
        q.num_inflight -= 1
        q.output_token_ids.append(7)
    rows = s.schedule_steady_decode()
    assert [q.request_id for q in rows] == ["a", "b"] and cache.num_free_pages() <= free
    for q in rows:
        q.num_computed_tokens += 1
        q.num_inflight += 1
    # a has 3 tokens now (one of them in flight): complete by length, not run again
    rows = s.schedule_steady_decode()
    assert [q.request_id for q in rows] == ["b"]
    # pages short: nothing is reserved and the general path must decide
    cache.admit("hog")
    assert cache.reserve("hog", 2 * cache.num_free_pages())
    b.num_computed_tokens += 1
    b.num_inflight -= 1
    b.output_token_ids.append(7)
    b.num_inflight += 1
    before = cache.num_free_pages()
    assert s.schedule_steady_decode() is None or cache.num_free_pages() == before
    cache.check()
