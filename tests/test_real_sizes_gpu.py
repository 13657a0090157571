"""The composed bfloat16 path at real layer sizes: Qwen2.5-7B's (hidden 3584, 28 heads on 4 kv heads,
head size 128, intermediate 18944, vocabulary 152064) and Qwen2.5-14B's (hidden 5120, 40 heads on 8,
intermediate 13824), two layers each, random weights filled on the device.

The tiny configurations cannot show what only these sizes have: 112 (or 160) partial sums of squares
per token handed from product to product, the gated tile image at an intermediate size of 18,944,
seven heads of a group packed into 128-row attention tiles, the choice between the engine's product
and the library's made per bucket of token counts at load, CUDA graphs at batch 8 and 64.  The same
cuts of the work as in test_replay_gpu.py, compared with the plain implementation run in float32 on
the same bfloat16-rounded weights; logits are asked for at a few dozen places so that the host side
stays in seconds.
"""
import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from helpers import Replayer, compare

pytestmark = pytest.mark.gpu

BASE = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 2, "vocab_size": 152064,
        "rope_theta": 1000000.0, "tie_word_embeddings": False, "use_sliding_window": False,
        "max_position_embeddings": 32768, "hidden_act": "silu", "initializer_range": 0.02}
SIZES = {"7b": dict(BASE, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944,
                    rms_norm_eps=1e-6),
         "14b": dict(BASE, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=13824,
                     rms_norm_eps=1e-5)}
SEED, PAGE, MAX_LEN = 5, 16, 512
_host_weights, _plain_rows = {}, {}


def host_weights(size):
    """name -> float32 array: the model's tensors as the random-weights mode defines them (bfloat16 values);
    test_random_init.py shows that the device kernel and the host's numpy give the same bits."""
    if size not in _host_weights:
        from vllm_cpp_b200.weights.random_init import random_tensor
        cfg = SIZES[size]
        out = {}
        for name, shape in plain.parameter_shapes(cfg).items():
            role = "gain" if name.endswith("norm.weight") else "bias" if name.endswith(".bias") else "matrix"
            t = random_tensor(name, shape, role, SEED, 0.02, 0.02, dtype=torch.bfloat16, device="cuda")
            out[name] = t.float().cpu().numpy()
        _host_weights[size] = out
    return _host_weights[size]


def want_rows(size, ids, rows):
    """The plain implementation's logits at ``rows`` of the sequence ``ids`` (kept: the modes share prompts)."""
    key = (size, tuple(ids), tuple(rows))
    if key not in _plain_rows:
        _plain_rows[key] = plain.forward(host_weights(size), SIZES[size], ids, dtype=np.float32, rows=list(rows))
    return _plain_rows[key]


def ids_of(n, seed):
    return np.random.default_rng(seed).integers(0, BASE["vocab_size"], size=n).tolist()


def some_rows(n, count, seed):
    """``count`` places of a sequence of n, the first and the last always among them."""
    rng = np.random.default_rng(seed)
    mid = rng.choice(np.arange(1, n - 1), size=min(count - 2, max(0, n - 2)), replace=False) if n > 2 else []
    return sorted({0, n - 1, *map(int, mid)})


MODES = ["tuned", "tcgen05", "library"]


@pytest.fixture(scope="module", params=[("7b", m) for m in MODES] + [("14b", "tuned")], ids=lambda p: f"{p[0]}-{p[1]}")
def engine(request):
    """(size, mode, cache, runner, graph runner).  Modes: the products chosen by the measurement at load
    (what serving runs), every few-token product pinned to the engine's tcgen05 kernel, every product
    on the library."""
    from vllm_cpp_b200 import EngineConfig
    from vllm_cpp_b200.csrc import ops
    from vllm_cpp_b200.engine import factory
    from vllm_cpp_b200.engine.runner import ModelRunner
    size, mode = request.param
    saved = dict(ops._linear_choice)
    ops._linear_choice.clear()
    if mode == "tcgen05":
        ops.set_linear_tuning(False)
    elif mode == "library":
        ops.set_tcgen05_linear(False)
    pages = 64 * 4 + 160
    ecfg = EngineConfig(load_format="random", model_config=SIZES[size], seed=SEED, dtype="bfloat16", block_size=PAGE,
                        num_gpu_blocks=pages, max_num_seqs=64, max_model_len=MAX_LEN, max_num_batched_tokens=512,
                        use_cuda_graphs=False)
    model, cache, runner = factory.build(ecfg)
    graphs = ModelRunner(model, cache, 512, 64, MAX_LEN, runner.device, use_cuda_graphs=True)
    yield size, mode, cache, runner, graphs
    ops.set_linear_tuning(True)
    ops.set_tcgen05_linear(True)
    ops._linear_choice.clear()
    ops._linear_choice.update(saved)
    del model, cache, runner, graphs
    torch.cuda.empty_cache()


def check(rp, size, rid, ids, rows, what):
    compare(rp.logits_of(rid, rows), want_rows(size, ids, rows), "bfloat16", f"{size} {what}")


def test_whole_prompt(engine):
    size, mode, cache, runner, _ = engine
    free = cache.num_free_pages()
    ids = ids_of(300, 1)
    rows = some_rows(300, 24, 2)
    rp = Replayer(runner, cache)
    rp.step([("w", ids, rows)], end=["w"])
    check(rp, size, "w", ids, rows, f"{mode} whole prompt")
    assert cache.num_free_pages() == free


def test_prompt_then_the_last_32_one_by_one(engine):
    size, mode, cache, runner, _ = engine
    ids = ids_of(300, 1)
    head = 300 - 32
    rp = Replayer(runner, cache)
    rp.step([("d", ids[:head], [head - 1])])
    for t in range(head, 300):
        rp.step([("d", ids[t:t + 1], [0])])
    rp.step([("x", [1, 2], [])], end=["d", "x"])
    rows = list(range(head - 1, 300))
    check(rp, size, "d", ids, rows, f"{mode} decode")


def test_portions_down_to_two_tokens(engine):
    size, mode, cache, runner, _ = engine
    ids = ids_of(300, 1)
    sizes = [7, 2, 13, 3, 2, 31, 16, 2, 5, 33, 2, 64, 17, 40, 2, 61]
    assert sum(sizes) == 300
    wanted = set(some_rows(300, 24, 3))
    rp = Replayer(runner, cache)
    at = 0
    for s in sizes:
        rp.step([("p", ids[at:at + s], [i for i in range(s) if at + i in wanted or i == s - 1 and s == 2])])
        at += s
    rp.step([("x", [3, 4], [])], end=["p", "x"])
    rows = sorted(p for (rid, p) in rp.rows if rid == "p")
    check(rp, size, "p", ids, rows, f"{mode} portions")


def test_four_requests_mixed_on_few_pages(engine):
    """Up to four live requests, portions of some beside decoded tokens of others, on so few pages that a
    new request gets the pages an earlier one gave back."""
    from test_replay_gpu import mixed_trace
    from vllm_cpp_b200.cache.manager import CacheManager
    from vllm_cpp_b200.engine.runner import ModelRunner
    size, mode, _, runner, _ = engine
    cfg = dict(SIZES[size])
    todo, steps = mixed_trace(cfg, seed=21, n_requests=6, live=4)
    keep = {rid: set(some_rows(len(ids), 10, 7)) for rid, ids, _ in todo}
    fed = {rid: 0 for rid, _, _ in todo}
    # a cache of its own with just enough pages for four requests of up to 120 tokens
    pages = 4 * (-(-120 // PAGE)) + 1
    cache = CacheManager(runner.model.cache_specs(), PAGE, pages, 8, runner.model.dtype, runner.device)
    runner = ModelRunner(runner.model, cache, 512, 8, MAX_LEN, runner.device)
    rp = Replayer(runner, cache)
    for entries, end in steps:
        cut = []
        for rid, toks, _ in entries:
            cut.append((rid, toks, [i for i in range(len(toks)) if fed[rid] + i in keep[rid]]))
            fed[rid] += len(toks)
        rp.step(cut, end)
    assert not cache.requests and cache.num_free_pages() == pages
    for rid, ids, _ in todo:
        check(rp, size, rid, ids, sorted(keep[rid]), f"{mode} mixed {rid}")


def test_one_large_step_of_portions_beside_decoded_tokens(engine):
    """More than 128 tokens in one step (the library's products, norm kernels, prefill attention) with three
    requests that decode in it and two that read portions of their prompts, one of them from the middle."""
    size, mode, cache, runner, _ = engine
    reqs = {f"m{i}": ids_of(n, 30 + i) for i, n in enumerate((90, 75, 120, 260, 180))}
    rp = Replayer(runner, cache)
    rp.step([("m0", reqs["m0"][:89], []), ("m1", reqs["m1"][:74], []), ("m2", reqs["m2"][:119], []),
             ("m3", reqs["m3"][:100], [99])])
    rp.step([("m0", reqs["m0"][89:], [0]), ("m3", reqs["m3"][100:260], [0, 77, 159]), ("m1", reqs["m1"][74:], [0]),
             ("m4", reqs["m4"][:180], [0, 1, 179]), ("m2", reqs["m2"][119:], [0])], end=list(reqs))
    check(rp, size, "m0", reqs["m0"], [89], f"{mode} big step m0")
    check(rp, size, "m1", reqs["m1"], [74], f"{mode} big step m1")
    check(rp, size, "m2", reqs["m2"], [119], f"{mode} big step m2")
    check(rp, size, "m3", reqs["m3"], [99, 100, 177, 259], f"{mode} big step m3")
    check(rp, size, "m4", reqs["m4"], [0, 1, 179], f"{mode} big step m4")


@pytest.mark.parametrize("batch", [8, 64])
def test_decode_under_cuda_graphs(engine, batch):
    """Decode steps at batch 8 and 64: launched directly, captured, then replayed (four steps), against
    the same steps through direct launches and against the plain implementation."""
    size, mode, cache, direct, graphs = engine
    lens = [int(x) for x in np.random.default_rng(batch).integers(17, 60, size=batch)]
    lens[0], lens[-1] = 16, 64                    # a request that starts a page, one that ends one
    steps = 4
    reqs = [ids_of(n + steps, 500 + batch + i) for i, n in enumerate(lens)]
    got = {}
    for tag, runner in (("g", graphs), ("d", direct)):
        rp = Replayer(runner, cache)
        names = [f"{tag}{batch}_{i}" for i in range(batch)]
        for lo in range(0, batch, 8):             # prompts in groups that fit a step's 512 tokens
            rp.step([(names[i], reqs[i][:lens[i]], []) for i in range(lo, min(batch, lo + 8))])
        for s in range(steps):
            rp.step([(names[i], [reqs[i][lens[i] + s]], [0]) for i in range(batch)])
        rp.step([(names[0], [1], [])], end=names)
        got[tag] = rp
    if graphs.use_cuda_graphs:
        assert any(k[0] == batch for k in graphs.graphs), "no step of this batch size was captured"
    for i in range(batch):
        rows = list(range(lens[i], lens[i] + steps))
        a = got["g"].logits_of(f"g{batch}_{i}", rows)
        b = got["d"].logits_of(f"d{batch}_{i}", rows)
        assert np.array_equal(a, b), f"{size} {mode} batch {batch} request {i}: replayed steps differ from direct launches"
    for i in sorted({0, 1, batch // 2, batch - 1}):
        rows = list(range(lens[i], lens[i] + steps))
        check(got["g"], size, f"g{batch}_{i}", reqs[i], rows, f"{mode} graphs batch {batch} request {i}")


def test_a_step_of_2048_tokens_with_portions_and_decoded_tokens(engine):
    """The shape the continuous-batching benchmark runs: a step at the token budget of 2,048 that holds two
    decoding requests, the end of one long prompt and the middle of another (what serving runs: the tuned
    products only)."""
    from vllm_cpp_b200.cache.manager import CacheManager
    from vllm_cpp_b200.engine.runner import ModelRunner
    size, mode, _, runner, _ = engine
    if mode != "tuned" or size != "7b":
        pytest.skip("one configuration is enough for this shape")
    pages, max_len = 4 * 130, 2048
    cache = CacheManager(runner.model.cache_specs(), PAGE, pages, 4, runner.model.dtype, runner.device)
    big = ModelRunner(runner.model, cache, 2048, 4, max_len, runner.device)
    reqs = {"a": ids_of(50, 71), "b": ids_of(33, 72), "c": ids_of(1400, 73), "d": ids_of(1700, 74)}
    rp = Replayer(big, cache)
    rp.step([("a", reqs["a"][:49], []), ("b", reqs["b"][:32], []), ("c", reqs["c"][:300], []), ("d", reqs["d"][:600], [])])
    # 1 + 1 + 1100 + 946 = 2048 tokens
    rp.step([("a", reqs["a"][49:], [0]), ("c", reqs["c"][300:], [0, 555, 1099]), ("b", reqs["b"][32:], [0]),
             ("d", reqs["d"][600:1546], [0, 400, 945])], end=["a", "b", "c", "d"])
    assert cache.num_free_pages() == pages
    check(rp, size, "a", reqs["a"], [49], "2048-token step a")
    check(rp, size, "b", reqs["b"], [32], "2048-token step b")
    check(rp, size, "c", reqs["c"], [300, 855, 1399], "2048-token step c")
    check(rp, size, "d", reqs["d"][:1546], [600, 1000, 1545], "2048-token step d")


@pytest.mark.parametrize("host", ["python", "cpp"])
def test_many_requests_on_few_pages_with_every_sampling_option(tmp_path, host):
    """Continuous batching at 7B layer sizes under pressure: 96 requests of mixed lengths on a sixth of the
    pages they would need together (so requests are preempted and recomputed), 32 at a time, 256 tokens a
    step, greedy, temperature, top-p and top-k rows side by side over the vocabulary of 152,064, decode steps
    of every batch size captured as graphs.  Two runs give the same tokens; every id is a real one; every
    request gets its length; nothing is left in the cache.  (This is the workload that showed a top-p draw
    returning id 2^20 - 1 on a flat row, and captured steps kept after a scratch buffer had moved.)"""
    import json
    cfg = SIZES["7b"]
    n_req, budget, seqs = 96, 256, 32
    rng = np.random.default_rng(12)
    lens, gens = rng.integers(8, 600, size=n_req), rng.integers(4, 80, size=n_req)
    pages = int(sum(-(-(int(a) + int(b)) // PAGE) for a, b in zip(lens, gens))) // 6
    prompts = [rng.integers(0, cfg["vocab_size"], size=int(n)).tolist() for n in lens]

    def options(i):
        return dict(max_tokens=int(gens[i]), temperature=0.8 if i % 3 else 0.0, top_p=0.9 if i % 5 == 0 else 1.0,
                    top_k=50 if i % 7 == 0 else -1, seed=1000 + i, ignore_eos=True)

    if host == "python":
        from vllm_cpp_b200 import EngineConfig, SamplingParams
        from vllm_cpp_b200.csrc import ops
        from vllm_cpp_b200.engine.llm_engine import Engine
        eng = Engine(EngineConfig(load_format="random", model_config=cfg, seed=SEED, dtype="bfloat16", block_size=PAGE,
                                  num_gpu_blocks=pages, max_num_seqs=seqs, max_model_len=1024, max_num_batched_tokens=budget,
                                  max_tokens_per_step=budget))

        def run():
            ids = [eng.add_request(p, SamplingParams(**options(i))) for i, p in enumerate(prompts)]
            outs = {i: [] for i in ids}
            while eng.has_pending_work():
                for o in eng.step():
                    outs[o.seq_id].extend(o.tokens)
            torch.cuda.synchronize()
            ops.check_status()
            return [outs[i] for i in ids]
        free, preemptions = (lambda: eng.cache.num_free_pages()), (lambda: eng.scheduler.num_preemptions)
    else:
        from vllm_cpp_b200.engine.cpp_host import CppEngine
        (tmp_path / "config.json").write_text(json.dumps(cfg))
        eng = CppEngine(str(tmp_path), dtype="bfloat16", block_size=PAGE, num_gpu_blocks=pages, max_num_seqs=seqs,
                        max_model_len=1024, max_num_batched_tokens=budget, max_tokens_per_step=budget,
                        load_format="random", seed=SEED)

        def run():
            return eng.generate(prompts, per_request=[options(i) for i in range(n_req)])
        free, preemptions = (lambda: eng.num_free_blocks), (lambda: eng.num_preemptions)
    first = run()
    assert preemptions() > 0
    second = run()
    assert first == second
    assert [len(t) for t in first] == [int(g) for g in gens]
    assert all(0 <= t < cfg["vocab_size"] for out in first for t in out)
    assert free() == pages


def test_captured_and_launched_ahead_steps_give_the_tokens_of_direct_launches_under_pressure():
    """The same workload as above on the Python host twice: decode steps captured as graphs and launched before
    the step before them has been read, and every kernel launched directly, one step at a time.  With the
    products' choice pinned (tune_products=False: what is measured at load may differ between two engines by
    timing noise, and then sums are taken in another order), both must sample the same tokens: a windowed layer, preemptions, greedy,
    temperature, top-p, top-k and repetition-penalty rows."""
    from vllm_cpp_b200 import EngineConfig, SamplingParams
    from vllm_cpp_b200.csrc import ops
    from vllm_cpp_b200.engine.llm_engine import Engine
    cfg = dict(SIZES["7b"], use_sliding_window=True, sliding_window=200, max_window_layers=1)
    n_req, budget, seqs = 60, 320, 24
    rng = np.random.default_rng(5)
    lens, gens = rng.integers(8, 700, size=n_req), rng.integers(4, 90, size=n_req)
    pages = int(sum(-(-(int(a) + int(b)) // PAGE) for a, b in zip(lens, gens))) // 5
    prompts = [rng.integers(0, cfg["vocab_size"], size=int(n)).tolist() for n in lens]

    def options(i):
        return dict(max_tokens=int(gens[i]), temperature=0.8 if i % 3 else 0.0, top_p=0.9 if i % 5 == 0 else 1.0,
                    top_k=50 if i % 7 == 0 else -1, repetition_penalty=1.2 if i % 11 == 0 else 1.0, seed=1000 + i, ignore_eos=True)

    results, shapes = {}, 0
    for fast in (True, False):
        eng = Engine(EngineConfig(load_format="random", model_config=cfg, seed=1, dtype="bfloat16", block_size=PAGE,
                                  num_gpu_blocks=pages, max_num_seqs=seqs, max_model_len=900, max_num_batched_tokens=budget,
                                  max_tokens_per_step=budget, use_cuda_graphs=fast, overlap_decode_steps=fast,
                                  tune_products=False))
        ids = [eng.add_request(p, SamplingParams(**options(i))) for i, p in enumerate(prompts)]
        outs = {i: [] for i in ids}
        while eng.has_pending_work():
            for o in eng.step():
                outs[o.seq_id].extend(o.tokens)
        torch.cuda.synchronize()
        ops.check_status()
        results[fast] = [outs[i] for i in ids]
        assert eng.scheduler.num_preemptions > 0 and eng.cache.num_free_pages() == pages
        if fast:
            shapes = len(eng.runner.graphs)
        del eng
    assert shapes >= 8
    differ = [i for i in range(n_req) if results[True][i] != results[False][i]]
    assert not differ, differ
