"""The C++ host's cache manager and scheduler beside the Python ones, decision for decision.

Random workloads (arrivals while others run, token budgets, pools from roomy to so tight that requests are
preempted and recomputed, windowed cache groups that give pages back, aborts) are stepped through both; every
step must schedule the same items (request, first position, count, whether a token is sampled), leave the same
number of free pages and the same block tables.  Runs without a GPU: the C++ side is src/cache.cpp built alone.
"""
import ctypes

import numpy as np
import pytest

from vllm_cpp_b200.cache.manager import CacheManager
from vllm_cpp_b200.csrc import build
from vllm_cpp_b200.engine.scheduler import Scheduler
from vllm_cpp_b200.engine.sequence import Sequence
from vllm_cpp_b200.parts.base import PagedKVSpec
from vllm_cpp_b200.sampling.params import SamplingParams


@pytest.fixture(scope="module")
def sim():
    l = ctypes.CDLL(build.build_scheduler_sim())
    P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    l.vcbs_create.argtypes, l.vcbs_create.restype = [P, I, I, I, I, I, I, I], P
    l.vcbs_destroy.argtypes = [P]
    l.vcbs_add_request.argtypes, l.vcbs_add_request.restype = [P, L, I, I], I
    l.vcbs_step.argtypes, l.vcbs_step.restype = [P, P, P, P, P, I], I
    l.vcbs_abort.argtypes = [P, L]
    l.vcbs_free_pages.argtypes, l.vcbs_free_pages.restype = [P], I
    l.vcbs_preemptions.argtypes, l.vcbs_preemptions.restype = [P], L
    l.vcbs_pending.argtypes, l.vcbs_pending.restype = [P], I
    l.vcbs_table.argtypes, l.vcbs_table.restype = [P, L, I, P, I], I
    l.vcbs_last_error.restype = ctypes.c_char_p
    return l


@pytest.mark.parametrize("seed", range(24))
def test_same_decisions_as_the_python_scheduler(sim, seed):
    rng = np.random.default_rng(seed)
    page = int(rng.choice([16, 32]))
    windows = [[0], [0], [0, 40], [24]][seed % 4]                      # cache groups: all keys, or the last W
    max_seqs = int(rng.integers(2, 7))
    budget = int(rng.choice([16, 48, 256]))
    portion = int(rng.choice([8, 24, 256]))
    n_req = 14
    lens = rng.integers(1, 140, size=n_req)
    outs = rng.integers(1, 40, size=n_req)
    longest = int((lens + outs).max())
    pages = int(rng.choice([-(-longest // page), -(-longest // page) + 3, 40]))       # tight, a little room, roomy
    to_front = bool(seed % 3 == 0)
    specs = [PagedKVSpec(1, 16, w) for w in windows]
    cache = CacheManager(specs, page, pages, max_seqs)
    py = Scheduler(cache, max_seqs, budget, portion, to_front)
    w = np.asarray(windows, dtype=np.int32)
    h = sim.vcbs_create(w.ctypes.data, len(windows), page, pages, max_seqs, budget, portion, 1 if to_front else 0)
    seqs = {}
    arrive = sorted(int(x) for x in rng.integers(0, 60, size=n_req))
    abort_at = {int(rng.integers(5, 80)): int(rng.integers(0, n_req)) for _ in range(2)}
    cap = 64
    ids, starts, counts, samples = (np.empty(cap, dtype=np.int64), np.empty(cap, dtype=np.int32), np.empty(cap, dtype=np.int32),
                                    np.empty(cap, dtype=np.int32))
    step, added = 0, 0
    while step < 2000:
        while added < n_req and arrive[added] <= step:
            s = Sequence(added, [1] * int(lens[added]), SamplingParams(max_tokens=int(outs[added])))
            try:
                py.add_request(s)
                ok = True
            except ValueError:
                ok = False
            assert (sim.vcbs_add_request(h, added, int(lens[added]), int(outs[added])) == 0) == ok
            if ok:
                seqs[added] = s
            added += 1
        if step in abort_at and abort_at[step] in seqs and not seqs[abort_at[step]].is_finished:
            py.abort_request(abort_at[step])
            sim.vcbs_abort(h, abort_at[step])
        items = py.schedule()
        n = sim.vcbs_step(h, ids.ctypes.data, starts.ctypes.data, counts.ctypes.data, samples.ctypes.data, cap)
        assert n >= 0, sim.vcbs_last_error()
        got = [(int(ids[i]), int(starts[i]), int(counts[i]), bool(samples[i])) for i in range(n)]
        assert got == [(it.seq.seq_id, it.start, it.count, it.samples) for it in items], f"step {step}"
        # the tables, before the step's commits change them on the Python side too
        for it in items:
            cache.commit(it.seq.seq_id, it.count)
            it.seq.num_processed_tokens += it.count
        for it in items:
            if it.samples:
                it.seq.output_tokens.append(7)
                if it.seq.output_len >= it.seq.params.max_tokens:
                    py.finish_sequence(it.seq, "length")
        assert sim.vcbs_free_pages(h) == cache.num_free_pages(), f"step {step}"
        buf = np.empty(64, dtype=np.int32)
        for s in py.running:
            for g in range(len(windows)):
                t = cache.table(s.seq_id, g)
                assert sim.vcbs_table(h, s.seq_id, g, buf.ctypes.data, 64) == len(t) and buf[:len(t)].tolist() == t
        assert sim.vcbs_preemptions(h) == py.num_preemptions
        assert bool(sim.vcbs_pending(h)) == py.has_pending_work()
        step += 1
        if added == n_req and not py.has_pending_work():
            break
    assert not py.has_pending_work() and cache.num_free_pages() == pages and sim.vcbs_free_pages(h) == pages
    sim.vcbs_destroy(h)
