"""The step function against the plain implementation under every way of cutting
the work: whole prompts; most of a prompt at once and the last 32 tokens one by
one; portions of changing size down to two tokens; and up to four live requests
mixed, prompt portions beside decoded tokens, with so few pages that pages are
used again.  In 32-bit and in bfloat16, on four tiny configurations.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_qwen2 as plain
from helpers import CONFIGS, Replayer, compare, make_weights, model_folder, token_ids

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build(tmp_path, name, dtype, num_pages, seed=1, max_seqs=8):
    from vllm_cpp_b200 import EngineConfig
    from vllm_cpp_b200.engine import factory
    cfg, page = CONFIGS[name]
    weights = make_weights(cfg, seed, dtype)
    folder = model_folder(tmp_path, cfg, weights, dtype)
    ecfg = EngineConfig(model_path=folder, dtype=dtype, block_size=page, num_gpu_blocks=num_pages,
                        max_num_seqs=max_seqs, max_model_len=cfg["max_position_embeddings"],
                        max_num_batched_tokens=1024, use_cuda_graphs=False)
    model, cache, runner = factory.build(ecfg)
    return cfg, weights, cache, runner


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_whole_prompts(tmp_path, name, dtype):
    cfg, weights, cache, runner = build(tmp_path, name, dtype, num_pages=40)
    rp = Replayer(runner, cache)
    for i, n in enumerate([1, 5, 17, 33, 100, 200]):
        ids = token_ids(cfg, n, 100 + i)
        rp.step([(f"r{i}", ids, range(n))], end=[f"r{i}"])
        compare(rp.logits_of(f"r{i}", range(n)), plain.forward(weights, cfg, ids), dtype, f"{name} whole n={n}")
    assert cache.num_free_pages() == 40


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_prefill_then_decode_last_32(tmp_path, name, dtype):
    cfg, weights, cache, runner = build(tmp_path, name, dtype, num_pages=40)
    rp = Replayer(runner, cache)
    for i, n in enumerate([40, 97, 180]):
        ids = token_ids(cfg, n, 200 + i)
        head = n - 32
        rp.step([("r", ids[:head], [head - 1])])
        for t in range(head, n):
            rp.step([("r", ids[t:t + 1], [0])])
        rp.step([("x", [1, 2], [])], end=["r", "x"])
        want = plain.forward(weights, cfg, ids)
        compare(rp.logits_of("r", range(head - 1, n)), want[head - 1:], dtype, f"{name} decode n={n}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_portions_of_changing_size(tmp_path, name, dtype):
    cfg, weights, cache, runner = build(tmp_path, name, dtype, num_pages=40)
    rp = Replayer(runner, cache)
    rng = np.random.default_rng(5)
    for i, n in enumerate([64, 150, 231]):
        ids = token_ids(cfg, n, 300 + i)
        cuts, at = [], 0
        sizes = [7, 2, 13, 3, 2, 31, 16, 2, 5, 33, 2, 64, 17]
        k = 0
        while at < n:
            s = min(sizes[k % len(sizes)] if i < 2 else int(rng.integers(2, 40)), n - at)
            if n - at - s == 1:          # never leave a single token: portions go down to two
                s += 1
            cuts.append((at, at + s))
            at += s
            k += 1
        for a, b in cuts:
            rp.step([("r", ids[a:b], range(b - a))])
        rp.step([("x", [3, 4], [])], end=["r", "x"])
        compare(rp.logits_of("r", range(n)), plain.forward(weights, cfg, ids), dtype, f"{name} portions n={n}")


def mixed_trace(cfg, seed, n_requests=7, live=4):
    """Steps of up to ``live`` requests: each request is cut into random portions (>= 2 tokens)
    and then decodes a few tokens one by one; a new request starts when one ends."""
    rng = np.random.default_rng(seed)
    todo = []
    for r in range(n_requests):
        n = int(rng.integers(20, 120))
        ids = token_ids(cfg, n, seed * 100 + r)
        n_dec = int(rng.integers(3, 12))
        cuts, at = [], 0
        while at < n - n_dec:
            s = min(int(rng.integers(2, 48)), n - n_dec - at)
            if n - n_dec - at - s == 1:
                s += 1
            cuts.append((at, at + s))
            at += s
        cuts += [(t, t + 1) for t in range(at, n)]
        todo.append((f"q{r}", ids, cuts))
    steps, running, nxt = [], [], 0
    while running or nxt < len(todo):
        while len(running) < live and nxt < len(todo):
            running.append([todo[nxt], 0])
            nxt += 1
        entries, end = [], []
        for item in running:
            (rid, ids, cuts), k = item
            if rng.random() < 0.2 and len(running) > 1:
                continue                      # a request may sit a step out
            a, b = cuts[k]
            entries.append((rid, ids[a:b], list(range(b - a))))
            item[1] += 1
            if item[1] == len(cuts):
                end.append(rid)
        running = [it for it in running if it[0][0] not in end]
        if entries:
            steps.append((entries, end))
    return todo, steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_mixed_requests_reusing_pages(tmp_path, name, dtype):
    cfg, page = CONFIGS[name]
    # four live requests of up to 120 tokens: just enough pages, so freed ones are reused at once
    pages = 4 * (-(-120 // page)) + 1
    cfg, weights, cache, runner = build(tmp_path, name, dtype, num_pages=pages)
    rp = Replayer(runner, cache)
    todo, steps = mixed_trace(cfg, seed=11)
    for entries, end in steps:
        rp.step(entries, end)
    assert cache.num_free_pages() == pages and not cache.requests
    for rid, ids, _ in todo:
        compare(rp.logits_of(rid, range(len(ids))), plain.forward(weights, cfg, ids), dtype, f"{name} mixed {rid}")


@pytest.fixture
def pinned_tcgen05():
    """Every bfloat16 product with few tokens on this library's tcgen05 kernel: nothing is measured at load."""
    from vllm_cpp_b200.csrc import ops
    saved = dict(ops._linear_choice)
    ops._linear_choice.clear()
    ops.set_linear_tuning(False)
    yield ops
    ops.set_linear_tuning(True)
    ops._linear_choice.update(saved)


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_norms_fused_into_products(tmp_path, pinned_tcgen05, name):
    """Steps of up to 128 tokens run no norm kernel between products: the product before a norm adds
    into the residual stream and applies the gain, the one after applies the rows' factor.  Portions,
    decoding and mixed steps against the plain implementation, and a count of the norm kernels left."""
    ops = pinned_tcgen05
    cfg, page = CONFIGS[name]
    cfg, weights, cache, runner = build(tmp_path, name, "bfloat16", num_pages=4 * (-(-120 // page)) + 1)
    assert all(b.mixer.fuses_norm(8) and b.feed_forward.fuses_norm(128) for b in runner.model.blocks)
    calls = []
    keep = ops.add_rmsnorm
    ops.add_rmsnorm = lambda *a, **k: (calls.append(1), keep(*a, **k))[1]
    try:
        rp = Replayer(runner, cache)
        ids = token_ids(cfg, 150, 41)
        rp.step([("r", ids[:100], range(100))])
        assert len(calls) == 2, "one norm after the embedding, one before the output product"
        rp.step([("r", ids[100:102], range(2))])
        for t in range(102, 150):
            rp.step([("r", ids[t:t + 1], [0])])
        rp.step([("x", [3, 4], [])], end=["r", "x"])
        compare(rp.logits_of("r", range(150)), plain.forward(weights, cfg, ids), "bfloat16", f"{name} fused norms")
        del calls[:]
        rp.step([("big", token_ids(cfg, 129, 42), [128])], end=["big"])     # above 128 tokens: the norm kernels run
        assert len(calls) == 2 * cfg["num_hidden_layers"] + 1
    finally:
        ops.add_rmsnorm = keep
    rp = Replayer(runner, cache)
    todo, steps = mixed_trace(cfg, seed=12)
    for entries, end in steps:
        rp.step(entries, end)
    for rid, ids, _ in todo:
        compare(rp.logits_of(rid, range(len(ids))), plain.forward(weights, cfg, ids), "bfloat16", f"{name} fused mixed {rid}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    """bin/trace_run as a user calls it: JSON lines in, <step>.f32 files and 'done' lines out."""
    cfg, page = CONFIGS["B"]
    weights = make_weights(cfg, 3, dtype)
    folder = model_folder(tmp_path, cfg, weights, dtype)
    ids_a, ids_b = token_ids(cfg, 70, 1), token_ids(cfg, 45, 2)
    lines = [
        {"step": 0, "entries": [{"id": "a", "tokens": ids_a[:50], "want": [0, 49]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": ids_a[50:52], "want": []},
                                {"id": "b", "tokens": ids_b[:30], "want": [29]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": ids_b[30:], "want": [14]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": ids_a[52:], "want": [17]},
                                {"id": "c", "tokens": ids_b, "want": [44]}], "end": ["a", "c"]},
    ]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                        "--out", str(out), "--max-tokens", "192"],
                       input="".join(json.dumps(l) + "\n" for l in lines), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    assert p.stdout.split() == ["done", "0", "done", "1", "done", "2", "done", "3"]
    want_a, want_b = plain.forward(weights, cfg, ids_a), plain.forward(weights, cfg, ids_b)
    v = cfg["vocab_size"]
    read = lambda s: np.fromfile(out / f"{s}.f32", dtype="<f4").reshape(-1, v)
    compare(read(0), want_a[[0, 49]], dtype, "trace step 0")
    compare(read(1), want_b[[29]], dtype, "trace step 1")
    compare(read(2), want_b[[44]], dtype, "trace step 2")
    compare(read(3), np.stack([want_a[69], want_b[44]]), dtype, "trace step 3")
