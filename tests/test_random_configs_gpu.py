"""Configurations drawn at random (head sizes in steps of 16, odd widths and vocabularies, any heads and
groups, windows, tied or not), each under a random mixed trace with so few pages that they are used again:
both hosts against the plain implementation, in 32-bit and in bfloat16.  The seeds are fixed, so a failure
names a configuration that can be run again."""
import numpy as np
import pytest

import plain_qwen2 as plain
from helpers import Replayer, compare, make_weights, model_folder, random_config
from test_replay_gpu import mixed_trace

pytestmark = pytest.mark.gpu


def drawn(seed):
    rng = np.random.default_rng(seed)
    cfg = random_config(rng)
    return cfg, int(rng.choice([16, 32, 64]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [7001, 7002, 7003, 7004, 7005, 7006])
def test_python_host_on_a_random_configuration(tmp_path, seed, dtype):
    from vllm_cpp_b200 import EngineConfig
    from vllm_cpp_b200.engine import factory
    cfg, page = drawn(seed)
    weights = make_weights(cfg, seed, dtype)
    folder = model_folder(tmp_path, cfg, weights, dtype)
    pages = 4 * (-(-120 // page)) + 1
    model, cache, runner = factory.build(EngineConfig(
        model_path=folder, dtype=dtype, block_size=page, num_gpu_blocks=pages, max_num_seqs=4,
        max_model_len=cfg["max_position_embeddings"], max_num_batched_tokens=512, use_cuda_graphs=False))
    rp = Replayer(runner, cache)
    todo, steps = mixed_trace(cfg, seed=seed, n_requests=6, live=4)
    for entries, end in steps:
        rp.step(entries, end)
    assert cache.num_free_pages() == pages and not cache.requests
    for rid, ids, _ in todo:
        compare(rp.logits_of(rid, range(len(ids))), plain.forward(weights, cfg, ids), dtype, f"seed {seed} {cfg} {rid}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [7101, 7102, 7103, 7104])
def test_cpp_host_on_a_random_configuration(tmp_path, seed, dtype):
    from test_cpp_host_gpu import CppReplayer
    from vllm_cpp_b200.engine.cpp_host import CppEngine
    cfg, page = drawn(seed)
    weights = make_weights(cfg, seed, dtype)
    folder = model_folder(tmp_path, cfg, weights, dtype)
    pages = 4 * (-(-120 // page)) + 1
    eng = CppEngine(folder, dtype=dtype, block_size=page, num_gpu_blocks=pages, max_num_seqs=4,
                    max_model_len=cfg["max_position_embeddings"], max_num_batched_tokens=512)
    rp = CppReplayer(eng)
    todo, steps = mixed_trace(cfg, seed=seed, n_requests=6, live=4)
    for entries, end in steps:
        rp.step(entries, end)
    assert eng.num_free_blocks == pages
    for rid, ids, _ in todo:
        compare(rp.logits_of(rid, range(len(ids))), plain.forward(weights, cfg, ids), dtype, f"seed {seed} {cfg} {rid}")
    eng.close()
