"""The scheduler's decisions, without a GPU.  Progress of the engine is faked the way the
reference's own scheduler test does it (tests/unit/test_scheduler.cpp:55,64-65,73): the
test advances ``num_processed_tokens`` and appends tokens by hand."""
import random

import pytest

from test_cache_manager import check_invariants
from vllm_cpp_b200.cache.manager import CacheManager
from vllm_cpp_b200.engine.scheduler import Scheduler
from vllm_cpp_b200.engine.sequence import Sequence, SequenceStatus
from vllm_cpp_b200.parts.base import PagedKVSpec
from vllm_cpp_b200.sampling.params import SamplingParams

FULL = PagedKVSpec(2, 16, 0)


def make(num_pages, page=16, max_seqs=8, batched=64, per_step=32, front=False):
    cache = CacheManager([FULL], page, num_pages, max_seqs)
    return cache, Scheduler(cache, max_seqs, batched, per_step, front)


def seq(i, n_prompt, max_tokens=8):
    return Sequence(i, list(range(1, n_prompt + 1)), SamplingParams(max_tokens=max_tokens), arrival=i)


def run_step(sched, cache, items, token=7):
    """What the engine does after a step."""
    for it in items:
        cache.commit(it.seq.seq_id, it.count)
        it.seq.num_processed_tokens += it.count
    for it in items:
        if it.samples:
            it.seq.output_tokens.append(token)
            if it.seq.output_len >= it.seq.params.max_tokens:
                sched.finish_sequence(it.seq, "length")


def test_admission_and_first_portion():
    cache, s = make(num_pages=8)
    a = seq(0, 16)
    s.add_request(a)
    assert s.has_pending_work() and a.status == SequenceStatus.WAITING
    items = s.schedule()
    # a prompt of 16 tokens takes one block of 16 (tests/unit/test_scheduler.cpp:27-38)
    assert [(i.seq.seq_id, i.start, i.count, i.samples) for i in items] == [(0, 0, 16, True)]
    assert a.status == SequenceStatus.RUNNING and len(cache.table(0, 0)) == 1 and len(s.waiting) == 0


def test_request_larger_than_the_pool_is_refused():
    cache, s = make(num_pages=2)
    with pytest.raises(ValueError, match="exceeds total KV cache block capacity"):
        s.add_request(seq(0, 30, max_tokens=8))
    with pytest.raises(ValueError, match="at least one token"):
        s.add_request(seq(1, 0))
    s.add_request(seq(2, 24, max_tokens=8))


def test_prompt_is_cut_under_the_token_budgets():
    cache, s = make(num_pages=32, batched=64, per_step=24)
    s.add_request(seq(0, 100, max_tokens=3))
    s.add_request(seq(1, 9, max_tokens=3))
    counts = []
    for _ in range(12):
        items = s.schedule()
        counts.append([(i.seq.seq_id, i.start, i.count) for i in items])
        assert sum(i.count for i in items if i.count > 1) <= 24 and sum(i.count for i in items) <= 64
        run_step(s, cache, items)
        if not s.has_pending_work():
            break
    assert counts[0] == [(0, 0, 24)]
    assert counts[1] == [(0, 24, 24)] and counts[2] == [(0, 48, 24)] and counts[3] == [(0, 72, 24)]
    # the last 4 prompt tokens leave 20 of the budget to the next request's whole prompt
    assert counts[4] == [(0, 96, 4), (1, 0, 9)]
    # both decode together now, decoding requests first
    assert counts[5] == [(0, 100, 1), (1, 9, 1)]
    assert not s.has_pending_work() and cache.num_free_pages() == 32


def test_decoding_requests_come_before_prompt_portions():
    cache, s = make(num_pages=32, batched=20, per_step=16)
    s.add_request(seq(0, 5, max_tokens=10))
    run_step(s, cache, s.schedule())
    s.add_request(seq(1, 40, max_tokens=2))
    items = s.schedule()
    assert [(i.seq.seq_id, i.count) for i in items] == [(0, 1), (1, 16)]
    run_step(s, cache, items)
    items = s.schedule()
    assert [(i.seq.seq_id, i.start, i.count) for i in items] == [(0, 6, 1), (1, 16, 16)]


def test_preempt_newest_and_requeue_when_decode_needs_a_page():
    # the reference's scenario (tests/unit/test_scheduler.cpp:47-89): 3 blocks of 16, two 16-token prompts
    cache, s = make(num_pages=3, batched=64, per_step=32)
    a, b = seq(0, 16, max_tokens=32), seq(1, 16, max_tokens=32)
    s.add_request(a)
    run_step(s, cache, s.schedule(), token=5)
    items = s.schedule()                                   # a decodes and takes its second block
    assert [(i.seq.seq_id, i.start, i.count) for i in items] == [(0, 16, 1)] and len(cache.table(0, 0)) == 2
    run_step(s, cache, items, token=5)
    s.add_request(b)
    items = s.schedule()
    assert [(i.seq.seq_id, i.count) for i in items] == [(0, 1), (1, 16)] and cache.num_free_pages() == 0
    run_step(s, cache, items, token=42)
    assert b.output_tokens == [42] and b.replay_len == 16
    # b needs a second block for its next token and nobody newer holds one: it sits steps out
    # while a, the older one, goes on inside its block
    for _ in range(14):
        items = s.schedule()
        assert [i.seq.seq_id for i in items] == [0] and b.status == SequenceStatus.RUNNING
        run_step(s, cache, items, token=6)
    b.output_tokens.append(43)                              # as in the reference's test
    assert b.replay_len == 17 and b.replay_token(16) == 42
    assert a.num_processed_tokens == 32
    # a reaches the next block boundary while b owns the last block: b is preempted and queued
    items = s.schedule()
    assert [(i.seq.seq_id, i.start, i.count) for i in items] == [(0, 32, 1)]
    assert b.status == SequenceStatus.PREEMPTED and b.needs_recompute and b.num_processed_tokens == 0
    assert 1 not in cache.requests and list(s.waiting) == [b] and s.running == [a]
    assert len(cache.table(0, 0)) == 3 and s.num_preemptions == 1
    check_invariants(cache)
    run_step(s, cache, items, token=6)
    s.finish_sequence(a, "abort")
    # b comes back: prompt and outputs are fed again as one portion, which ends in a sampled token
    items = s.schedule()
    assert [(i.seq.seq_id, i.start, i.count, i.samples) for i in items] == [(1, 0, 18, True)]
    assert len(cache.table(1, 0)) == 2 and not b.needs_recompute and b.status == SequenceStatus.RUNNING
    run_step(s, cache, items, token=9)
    assert b.output_tokens == [42, 43, 9]


def test_preempted_request_goes_to_the_front_or_the_back():
    for front in (True, False):
        cache, s = make(num_pages=2, front=front)
        a, b, c = seq(0, 15, 8), seq(1, 14, 8), seq(2, 20, 1)
        s.add_request(a); s.add_request(b)
        run_step(s, cache, s.schedule())
        s.add_request(c)                                    # cannot be admitted: no page
        run_step(s, cache, s.schedule())                    # a: 16 tokens, b: 15
        assert s.num_preemptions == 0
        s.schedule()                                        # a needs a second page: b gives its page
        assert b.status == SequenceStatus.PREEMPTED
        assert list(s.waiting) == ([b, c] if front else [c, b])


def test_waiting_request_never_preempts():
    cache, s = make(num_pages=4, batched=64, per_step=64)
    a = seq(0, 40, max_tokens=8)
    s.add_request(a)
    run_step(s, cache, s.schedule())
    s.add_request(seq(1, 30, max_tokens=2))         # needs 2 pages, 1 is free
    items = s.schedule()
    assert [i.seq.seq_id for i in items] == [0] and a.status == SequenceStatus.RUNNING
    assert len(s.waiting) == 1 and s.num_preemptions == 0


def test_stalled_prompts_are_untangled():
    # two prompts that each need most of the pool are both admitted portion by portion,
    # fill it, and neither decodes: the newer one gives way
    cache, s = make(num_pages=6, batched=64, per_step=32)
    a, b = seq(0, 80, max_tokens=2), seq(1, 80, max_tokens=2)
    s.add_request(a); s.add_request(b)
    done = 0
    for _ in range(40):
        items = s.schedule()
        assert items, "the scheduler stalled"
        run_step(s, cache, items)
        check_invariants(cache)
        if not s.has_pending_work():
            break
    assert a.is_finished and b.is_finished and s.num_preemptions >= 1 and cache.num_free_pages() == 6


def test_abort_and_slots():
    cache, s = make(num_pages=8, max_seqs=2)
    for i in range(3):
        s.add_request(seq(i, 4))
    items = s.schedule()
    assert [i.seq.seq_id for i in items] == [0, 1] and len(s.waiting) == 1     # max_num_seqs
    run_step(s, cache, items)
    assert s.abort_request(0) and not s.abort_request(77)
    assert cache.num_free_pages() == 7
    assert [i.seq.seq_id for i in s.schedule()] == [1, 2]
    assert s.abort_request(2) and s.abort_request(1) and not s.has_pending_work()
    assert cache.num_free_pages() == 8


@pytest.mark.parametrize("seed", range(4))
def test_random_load_finishes_everything(seed):
    rng = random.Random(seed)
    cache, s = make(num_pages=12, max_seqs=4, batched=48, per_step=24)
    seqs = []
    for step in range(400):
        if rng.random() < 0.15 and len(seqs) < 25:
            q = seq(len(seqs), rng.randint(1, 90), max_tokens=rng.randint(1, 20))
            s.add_request(q)
            seqs.append(q)
        items = s.schedule()
        ids = [i.seq.seq_id for i in items]
        assert len(ids) == len(set(ids)) and sum(i.count for i in items) <= 48
        for i in items:
            assert i.start == i.seq.num_processed_tokens == cache.num_tokens(i.seq.seq_id)
            assert i.samples == (i.start + i.count == i.seq.total_len)
        run_step(s, cache, items, token=rng.randint(0, 9))
        check_invariants(cache)
    while s.has_pending_work():
        items = s.schedule()
        assert items
        run_step(s, cache, items)
    assert all(q.is_finished and q.output_len == q.params.max_tokens for q in seqs)
    assert cache.num_free_pages() == 12 and not cache.requests
