"""Generation through the Python entry point against the plain implementation:
greedy and seeded sampling, requests alone and together, under a small token budget,
and with so few pages that requests are preempted and recomputed."""
import numpy as np
import pytest

import plain_qwen2 as plain
from helpers import CONFIGS, make_weights, model_folder, token_ids

pytestmark = pytest.mark.gpu


def check_greedy(weights, cfg, prompt, out, dtype):
    """Every generated token must be the plain implementation's choice given the tokens before
    it, or lie within the logits' tolerance of that choice (a near tie decided by rounding)."""
    from helpers import TOL
    ids = list(prompt)
    exact = 0
    for tok in out:
        logits = plain.forward(weights, cfg, ids)[-1]
        best = plain.greedy(logits)
        gap = (logits[best] - logits[tok]) / np.abs(logits).max()
        assert gap <= 2 * TOL[dtype], f"token {tok} instead of {best}: gap {gap:.3e} after {len(ids)} tokens"
        exact += tok == best
        ids.append(tok)
    return exact


def make_llm(tmp_path, name, dtype, **kw):
    from vllm_cpp_b200 import LLM
    cfg, page = CONFIGS[name]
    weights = make_weights(cfg, 21, dtype)
    folder = model_folder(tmp_path, cfg, weights, dtype)
    args = dict(dtype=dtype, block_size=page, num_gpu_blocks=64, max_num_seqs=8,
                max_model_len=cfg["max_position_embeddings"], max_num_batched_tokens=256)
    args.update(kw)
    return cfg, weights, LLM(folder, **args)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("C", "float32"), ("A", "bfloat16"),
                                        ("D", "bfloat16")])
def test_greedy_generation_matches_plain(tmp_path, name, dtype):
    from vllm_cpp_b200 import SamplingParams
    cfg, weights, llm = make_llm(tmp_path, name, dtype)
    prompts = [token_ids(cfg, n, 50 + n) for n in (5, 17, 33)]       # the tiny workload of configuration A
    outs = llm.generate(prompts, SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))
    exact = sum(check_greedy(weights, cfg, p, o, dtype) for p, o in zip(prompts, outs))
    assert all(len(o) == 8 for o in outs) and exact >= 20       # near ties are rare
    assert not llm.engine.has_pending_work() and llm.engine.cache.num_free_pages() == 64


def test_alone_together_budgeted_and_preempted_give_the_same_tokens(tmp_path):
    """Configuration B's workload: prompts 1, 9, 40, 64, 100; a 24-token budget; temperature 0.8
    with a fixed seed; 12 tokens each.  The draw is keyed by request seed and token index, so
    the tokens may not depend on batching, on the budget or on preemption."""
    from vllm_cpp_b200 import SamplingParams
    name, dtype = "B", "float32"
    cfg, _ = CONFIGS[name]
    prompts = [token_ids(cfg, n, 70 + n) for n in (1, 9, 40, 64, 100)]
    params = [SamplingParams(max_tokens=12, temperature=0.8, seed=1000 + i, ignore_eos=True) for i in range(5)]
    _, weights, llm = make_llm(tmp_path, name, dtype)
    alone = [llm.generate([p], sp)[0] for p, sp in zip(prompts, params)]
    together = llm.generate(prompts, params)
    _, _, budgeted = make_llm(tmp_path, name, dtype, max_tokens_per_step=24, max_num_batched_tokens=32)
    cut = budgeted.generate(prompts, params)
    # 7 pages of 32: the five requests need 9 at their longest, so some are preempted and recomputed
    _, _, small = make_llm(tmp_path, name, dtype, num_gpu_blocks=7, max_tokens_per_step=24)
    squeezed = small.generate(prompts, params)
    assert small.engine.scheduler.num_preemptions > 0
    assert together == alone and cut == alone and squeezed == alone
    assert all(len(o) == 12 for o in alone)
    # and the first sampled token of each is what the plain sampler draws from the plain logits
    from vllm_cpp_b200.sampling.sampler import uniform_for
    for p, sp, o in zip(prompts, params, alone):
        logits = plain.forward(weights, cfg, p)[-1]
        assert o[0] == plain.sample(logits, 0.8, 1.0, -1, 1.0, [], uniform_for(sp.seed, 0))


def test_stop_token_and_length(tmp_path):
    from vllm_cpp_b200 import SamplingParams
    cfg, weights, llm = make_llm(tmp_path, "A", "float32")
    p = token_ids(cfg, 12, 3)
    free = llm.generate([p], SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True))[0]
    stop = free[3]
    out = llm.generate([p], SamplingParams(max_tokens=10, temperature=0.0, stop_token_ids=[stop]))[0]
    assert out == free[:free.index(stop) + 1]
    with pytest.raises(ValueError, match="context length"):
        llm.generate([list(range(10))], SamplingParams(max_tokens=10_000))
    with pytest.raises(ValueError, match="vocabulary"):
        llm.generate([[cfg["vocab_size"]]], SamplingParams(max_tokens=1))
    with pytest.raises(ValueError, match="at least one token"):
        llm.generate([[]], SamplingParams(max_tokens=1))


def test_steps_launched_ahead_give_the_same_tokens(tmp_path):
    """With overlap_decode_steps the engine launches a step before it has read the step before it.
    Requests that stop at different times (stop token, length), a request that arrives while others
    decode and one that is aborted: the same tokens as with the option off, nothing left behind."""
    from vllm_cpp_b200 import SamplingParams
    cfg, _ = CONFIGS["B"]
    prompts = [token_ids(cfg, n, 90 + n) for n in (3, 20, 41, 7)]
    runs = {}
    for overlap in (False, True):
        _, _, llm = make_llm(tmp_path, "B", "float32", overlap_decode_steps=overlap)
        eng = llm.engine
        free = llm.generate(prompts[:1], SamplingParams(max_tokens=24, temperature=0.7, seed=5, ignore_eos=True))[0]
        params = [SamplingParams(max_tokens=24, temperature=0.7, seed=5, stop_token_ids=[free[9]]),      # stops early
                  SamplingParams(max_tokens=30, temperature=0.0, ignore_eos=True),
                  SamplingParams(max_tokens=11, temperature=1.1, seed=9, top_k=20, ignore_eos=True),
                  SamplingParams(max_tokens=16, temperature=0.0, ignore_eos=True)]
        ids = [eng.add_request(p, sp) for p, sp in zip(prompts[:3], params[:3])]
        got = {i: [] for i in ids}
        aborted, steps, ahead_seen = None, 0, 0
        while eng.has_pending_work():
            for o in eng.step():
                got[o.seq_id].extend(o.tokens)
            steps += 1
            ahead_seen += eng._ahead is not None
            if steps == 6:                               # arrives while the others decode
                late = eng.add_request(prompts[3], params[3])
                got[late] = []
            if steps == 14:
                aborted = ids[1]
                eng.abort_request(aborted)
        assert -1 not in sum(got.values(), []), "a placeholder reached the caller"
        assert (ahead_seen > 5) == overlap
        assert eng.cache.num_free_pages() == 64 and not eng.cache.requests
        runs[overlap] = [got[ids[0]], got[ids[1]], got[ids[2]], got[late]]
    off, on = runs[False], runs[True]
    # the aborted request (second) may have got a token more or less before the abort took hold
    n = min(len(off[1]), len(on[1]))
    assert off[1][:n] == on[1][:n] and abs(len(off[1]) - len(on[1])) <= 1
    assert len(off[0]) == 10 and off[0] == on[0] and len(off[2]) == 11 and off[2] == on[2]
    assert len(off[3]) == 16 and off[3] == on[3]


@pytest.mark.parametrize("name", ["D", "E"])
def test_captured_steps_with_mixed_contexts_give_the_same_tokens(tmp_path, name):
    """Requests whose contexts differ twentyfold decode together on the tensor-core kernels: the splits of
    the decode attention follow the contexts and change the grid as they grow and as requests leave, and
    every such shape is captured as a graph of its own.  Same tokens as with every kernel launched
    directly, several shapes seen, nothing left behind."""
    from vllm_cpp_b200 import SamplingParams
    cfg, page = CONFIGS[name]
    prompts = [token_ids(cfg, n, 30 + n) for n in (250, 12, 90, 3, 180)]
    params = [SamplingParams(max_tokens=n, temperature=0.0, ignore_eos=True) for n in (40, 60, 25, 60, 33)]
    runs, shapes = {}, set()
    for graphs in (False, True):
        _, _, llm = make_llm(tmp_path, name, "bfloat16", use_cuda_graphs=graphs, num_gpu_blocks=96)
        eng = llm.engine
        ids = [eng.add_request(p, sp) for p, sp in zip(prompts, params)]
        got = {i: [] for i in ids}
        while eng.has_pending_work():
            for o in eng.step():
                got[o.seq_id].extend(o.tokens)
        runs[graphs] = [got[i] for i in ids]
        if graphs:
            shapes = set(eng.runner.graphs)
        assert eng.cache.num_free_pages() == 96 and not eng.cache.requests
    assert runs[False] == runs[True] and [len(t) for t in runs[True]] == [40, 60, 25, 60, 33]
    assert len(shapes) >= 3, shapes


def test_long_decoding_stays_on_the_plain_logits(tmp_path):
    """160 tokens decoded one by one after a 3-token prompt, replayed against the plain logits."""
    from vllm_cpp_b200.engine.runner import StepEntry
    for name, dtype in (("A", "float32"), ("C", "bfloat16")):
        cfg, weights, llm = make_llm(tmp_path, name, dtype)
        eng = llm.engine
        ids = token_ids(cfg, 163, 9)
        eng.cache.add_request("long")
        rows = [eng.runner.step([StepEntry("long", ids[:3], [0, 1, 2])]).float().cpu().numpy()]
        for t in range(3, len(ids)):
            rows.append(eng.runner.step([StepEntry("long", ids[t:t + 1], [0])]).float().cpu().numpy())
        eng.cache.free_request("long")
        from helpers import compare
        compare(np.concatenate(rows), plain.forward(weights, cfg, ids), dtype, f"{name} long decode")


@pytest.mark.parametrize("name", ["D", "E"])
def test_preemption_under_captured_steps_in_bfloat16(tmp_path, name):
    """bfloat16, CUDA graphs, steps launched ahead, and so few pages that running requests are preempted
    and recomputed while others decode: every generated token is the plain implementation's choice given
    the tokens before it (or within rounding of it), every request gets its full length, nothing is left
    behind, and the requests that were never preempted get the tokens they get with plenty of pages."""
    from vllm_cpp_b200 import SamplingParams
    cfg, page = CONFIGS[name]
    prompts = [token_ids(cfg, n, 60 + n) for n in (70, 9, 45, 120, 30)]
    sp = SamplingParams(max_tokens=48, temperature=0.0, ignore_eos=True)
    need = [-(-(len(p) + 48) // page) for p in prompts]
    _, weights, roomy = make_llm(tmp_path, name, "bfloat16", use_cuda_graphs=True, num_gpu_blocks=sum(need) + 2)
    plenty = roomy.generate(prompts, sp)
    assert roomy.engine.scheduler.num_preemptions == 0
    # room for all the prompts and one page more: every request is admitted, and as they grow the newest are
    # preempted and recomputed
    _, _, tight = make_llm(tmp_path, name, "bfloat16", use_cuda_graphs=True,
                           num_gpu_blocks=sum(-(-len(p) // page) for p in prompts) + 1)
    eng = tight.engine
    ids = [eng.add_request(p, sp) for p in prompts]
    got = {i: [] for i in ids}
    while eng.has_pending_work():
        for o in eng.step():
            got[o.seq_id].extend(o.tokens)
    assert eng.scheduler.num_preemptions > 0 and eng.runner.graphs, "the run must preempt and must replay graphs"
    assert not eng.cache.requests and eng.cache.num_free_pages() == eng.cache.num_pages
    for i, p, ref in zip(ids, prompts, plenty):
        assert len(got[i]) == 48
        check_greedy(weights, cfg, p, got[i], "bfloat16")
        # same tokens as with plenty of pages up to the first near tie that rounding decided otherwise
        same = next((k for k, (x, y) in enumerate(zip(got[i], ref)) if x != y), 48)
        assert same >= 8, f"request {i} leaves the roomy run's tokens after {same}"


def test_a_scratch_buffer_that_moves_makes_captured_steps_stale(tmp_path):
    """A captured step holds the addresses of the kernels' scratch buffers.  When a later step, launched
    directly because its shape is new, makes one of them grow, every graph captured before must go: the old
    memory is given back to the driver at the next capture.  Here the growth is forced inside the first run
    of a new shape; the graphs of the old shapes must be gone afterwards, and the old shapes must still give
    the plain implementation's tokens when they come again."""
    from vllm_cpp_b200 import SamplingParams
    from vllm_cpp_b200.csrc import ops
    cfg, weights, llm = make_llm(tmp_path, "E", "bfloat16", use_cuda_graphs=True, num_gpu_blocks=96)
    eng, runner = llm.engine, llm.engine.runner
    sp = SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True)
    prompts = [token_ids(cfg, n, 70 + n) for n in (40, 41, 42)]

    def generate(some):
        ids = [eng.add_request(p, sp) for p in some]
        got = {i: [] for i in ids}
        while eng.has_pending_work():
            for o in eng.step():
                got[o.seq_id].extend(o.tokens)
        return [got[i] for i in ids]

    first = generate(prompts[:2])                       # two requests: their decode shape is captured
    before = {k: g for k, g in runner.graphs.items()}
    assert before
    forward, grown = runner.model.forward, []

    def forward_that_grows_a_buffer(*a, **kw):
        if not grown and not __import__("torch").cuda.is_current_stream_capturing():
            grown.append(ops.scratch("attn_part_o", ops._scratch["attn_part_o"].numel() * 2 + 1, "cuda"))
        return forward(*a, **kw)

    runner.model.forward = forward_that_grows_a_buffer
    try:
        generate(prompts)                               # three requests: a new shape, whose first run moves the buffer
    finally:
        runner.model.forward = forward
    assert grown
    assert all(runner.graphs.get(k) is not g for k, g in before.items()), "a graph captured before the buffer moved is still there"
    again = generate(prompts[:2])
    assert again == first
    for p, out in zip(prompts[:2], again):
        check_greedy(weights, cfg, p, out, "bfloat16")


def test_captured_steps_are_bounded_in_number(tmp_path, monkeypatch):
    """Only so many captured steps are kept; the least recently replayed goes first and is captured again when
    its shape returns.  With room for two, a run that sees several shapes gives the tokens of direct launches."""
    import vllm_cpp_b200.engine.runner as runner_module
    from vllm_cpp_b200 import SamplingParams
    monkeypatch.setattr(runner_module, "MAX_CAPTURED_STEPS", 2)
    cfg, page = CONFIGS["E"]
    prompts = [token_ids(cfg, n, 30 + n) for n in (250, 12, 90, 3, 180)]
    params = [SamplingParams(max_tokens=n, temperature=0.0, ignore_eos=True) for n in (40, 60, 25, 60, 33)]
    runs = {}
    for graphs in (False, True):
        _, _, llm = make_llm(tmp_path, "E", "bfloat16", use_cuda_graphs=graphs, num_gpu_blocks=96)
        eng = llm.engine
        ids = [eng.add_request(p, sp) for p, sp in zip(prompts, params)]
        got = {i: [] for i in ids}
        most = 0
        while eng.has_pending_work():
            for o in eng.step():
                got[o.seq_id].extend(o.tokens)
            most = max(most, len(eng.runner.graphs))
        runs[graphs] = [got[i] for i in ids]
        if graphs:
            assert most == 2
    assert runs[False] == runs[True]
