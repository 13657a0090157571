"""The C++ host runtime (include/vllm/vllm.hpp, src/) against the plain implementation and against the
Python host: explicit batches cut every way, the two tiny workloads under its scheduler with the same token
ids as the Python engine, preemption, its loader's errors, its pool, its command line."""
import os
import subprocess

import numpy as np
import pytest

import plain_qwen2 as plain
from helpers import CONFIGS, compare, make_weights, model_folder, token_ids

pytestmark = pytest.mark.gpu


class CppReplayer:
    """helpers.Replayer for the C++ host: request names become small integers."""

    def __init__(self, eng):
        self.eng, self.fed, self.rows, self.ids = eng, {}, {}, {}

    def step(self, entries, end=()):
        batch = []
        for rid, toks, want in entries:
            if rid not in self.ids:
                self.ids[rid] = len(self.ids)
                self.fed[rid] = 0
            batch.append((self.ids[rid], list(toks), list(want)))
        logits = self.eng.step_tokens(batch)
        i = 0
        for rid, toks, want in entries:
            for w in want:
                self.rows[(rid, self.fed[rid] + w)] = logits[i].copy()
                i += 1
            self.fed[rid] += len(toks)
        for rid in end:
            self.eng.release(self.ids[rid])

    def logits_of(self, rid, positions):
        return np.stack([self.rows[(rid, p)] for p in positions])


def cpp_engine(tmp_path, name, dtype, seed=1, **kw):
    from vllm_cpp_b200.engine.cpp_host import CppEngine
    cfg, page = CONFIGS[name]
    weights = make_weights(cfg, seed, dtype)
    folder = model_folder(tmp_path, cfg, weights, dtype)
    args = dict(dtype=dtype, block_size=page, num_gpu_blocks=40, max_num_seqs=8, max_model_len=cfg["max_position_embeddings"],
                max_num_batched_tokens=1024)
    args.update(kw)
    return cfg, weights, folder, CppEngine(folder, **args)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "bfloat16-plain"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_explicit_batches_cut_every_way(tmp_path, name, dtype):
    """bfloat16: steps of up to 64 tokens run with the norms, additions and SwiGLU inside the products;
    "bfloat16-plain" switches that off, so every step runs the plain sequence of kernels."""
    from test_replay_gpu import mixed_trace
    cfg, page = CONFIGS[name]
    pages = 4 * (-(-120 // page)) + 1
    fused = dtype != "bfloat16-plain"
    dtype = dtype.split("-")[0]
    cfg, weights, _, eng = cpp_engine(tmp_path, name, dtype, num_gpu_blocks=max(pages, -(-231 // page) + 1), fused_decode_tokens=64 if fused else 0)
    total = eng.num_total_blocks
    assert 0 < eng.pool_used_bytes <= eng.pool_total_bytes
    rp = CppReplayer(eng)
    # whole, then most of it at once and the last 32 one by one
    ids = token_ids(cfg, 150, 300)
    rp.step([("w", ids, range(150))], end=["w"])
    compare(rp.logits_of("w", range(150)), plain.forward(weights, cfg, ids), dtype, f"{name} whole")
    rp.step([("d", ids[:118], [117])])
    for t in range(118, 150):
        rp.step([("d", ids[t:t + 1], [0])])
    rp.step([("x", [1, 2], [])], end=["d", "x"])
    compare(rp.logits_of("d", range(117, 150)), plain.forward(weights, cfg, ids)[117:], dtype, f"{name} decode")
    # portions down to two tokens
    ids = token_ids(cfg, 231, 301)
    at = 0
    for s in [7, 2, 13, 3, 2, 31, 16, 2, 5, 33, 2, 64, 17, 34]:
        rp.step([("p", ids[at:at + s], range(s))])
        at += s
    assert at == 231
    rp.step([("y", [3, 4], [])], end=["p", "y"])
    compare(rp.logits_of("p", range(231)), plain.forward(weights, cfg, ids), dtype, f"{name} portions")
    assert eng.num_free_blocks == total
    # four live requests mixed, pages used again
    todo, steps = mixed_trace(cfg, seed=11)
    for entries, end in steps:
        rp.step(entries, end)
    assert eng.num_free_blocks == total
    for rid, ids, _ in todo:
        compare(rp.logits_of(rid, range(len(ids))), plain.forward(weights, cfg, ids), dtype, f"{name} mixed {rid}")


def python_llm(folder, name, dtype, **kw):
    from vllm_cpp_b200 import LLM
    cfg, page = CONFIGS[name]
    args = dict(dtype=dtype, block_size=page, num_gpu_blocks=64, max_num_seqs=8, max_model_len=cfg["max_position_embeddings"],
                max_num_batched_tokens=256)
    args.update(kw)
    return LLM(folder, **args)


def test_the_tiny_workloads_give_the_same_tokens_on_both_hosts(tmp_path):
    """Configuration A: prompts 5, 17, 33, greedy, 8 tokens.  Configuration B: prompts 1, 9, 40, 64, 100, a
    24-token budget mixed with decoding, temperature 0.8 with fixed seeds, 12 tokens; and once more on so few
    pages that requests are preempted and recomputed.  float32: both hosts launch the same kernels."""
    from vllm_cpp_b200 import SamplingParams
    cfg, weights, folder, eng = cpp_engine(tmp_path, "A", "float32", seed=21, num_gpu_blocks=64, max_num_batched_tokens=256)
    prompts = [token_ids(cfg, n, 50 + n) for n in (5, 17, 33)]
    got = eng.generate(prompts, max_tokens=8, temperature=0.0, ignore_eos=True)
    want = python_llm(folder, "A", "float32").generate(prompts, SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))
    assert got == want and all(len(o) == 8 for o in got)
    assert eng.num_free_blocks == 64 and not eng.has_pending_work()
    eng.close()

    cfg, weights, folder, eng = cpp_engine(tmp_path, "B", "float32", seed=21, num_gpu_blocks=64, max_num_batched_tokens=32,
                                           max_tokens_per_step=24)
    prompts = [token_ids(cfg, n, 70 + n) for n in (1, 9, 40, 64, 100)]
    per = [dict(max_tokens=12, temperature=0.8, seed=1000 + i, ignore_eos=True) for i in range(5)]
    got = eng.generate(prompts, per_request=per)
    params = [SamplingParams(max_tokens=12, temperature=0.8, seed=1000 + i, ignore_eos=True) for i in range(5)]
    want = python_llm(folder, "B", "float32", max_tokens_per_step=24, max_num_batched_tokens=32).generate(prompts, params)
    assert got == want and all(len(o) == 12 for o in got)
    eng.close()
    # 7 pages of 32: the five requests need 9 at their longest
    _, _, _, small = cpp_engine(tmp_path, "B", "float32", seed=21, num_gpu_blocks=7, max_tokens_per_step=24)
    squeezed = small.generate(prompts, per_request=per)
    assert small.num_preemptions > 0 and squeezed == want and small.num_free_blocks == 7
    # top-k, top-p and the repetition penalty take the same path on both hosts
    per = [dict(max_tokens=10, temperature=1.1, top_k=20, top_p=0.9, repetition_penalty=1.3, seed=7 + i, ignore_eos=True) for i in range(5)]
    params = [SamplingParams(max_tokens=10, temperature=1.1, top_k=20, top_p=0.9, repetition_penalty=1.3, seed=7 + i, ignore_eos=True)
              for i in range(5)]
    _, _, _, eng = cpp_engine(tmp_path, "B", "float32", seed=21, num_gpu_blocks=64)
    assert eng.generate(prompts, per_request=per) == python_llm(folder, "B", "float32").generate(prompts, params)


def test_stop_tokens_abort_and_refusals(tmp_path):
    from vllm_cpp_b200.engine.cpp_host import CppEngineError
    cfg, weights, folder, eng = cpp_engine(tmp_path, "A", "float32", seed=21, num_gpu_blocks=64)
    p = token_ids(cfg, 12, 3)
    free = eng.generate([p], max_tokens=10, temperature=0.0, ignore_eos=True)[0]
    stop = free[3]
    assert eng.generate([p], max_tokens=10, temperature=0.0, stop_token_ids=[stop])[0] == free[:free.index(stop) + 1]
    a = eng.add_request(p, max_tokens=50, temperature=0.0, ignore_eos=True)
    b = eng.add_request(p, max_tokens=5, temperature=0.0, ignore_eos=True)
    eng.step(); eng.step()
    eng.abort_request(a)
    seen = []
    while eng.has_pending_work():
        seen += eng.step()
    assert {r for r, _, _ in seen} == {b} and seen[-1][2] == "length" and eng.num_free_blocks == 64
    for bad, msg in (([], "at least one token"), ([cfg["vocab_size"]], "vocabulary"), (list(range(10)) * 40, "context length")):
        with pytest.raises(CppEngineError, match=msg):
            eng.add_request(bad, max_tokens=4)
    with pytest.raises(CppEngineError, match="context length"):
        eng.add_request([1, 2, 3], max_tokens=10_000)
    with pytest.raises(CppEngineError, match="appears twice"):
        eng.step_tokens([(0, [1], []), (0, [2], [])])


def test_loader_and_configuration_errors(tmp_path):
    import json
    from vllm_cpp_b200.engine.cpp_host import CppEngine, CppEngineError
    cfg, page = CONFIGS["B"]
    w = make_weights(cfg, 0, "float32")
    broken = dict(w)
    del broken["model.layers.1.mlp.up_proj.weight"], broken["lm_head.weight"]
    broken["model.layers.9.extra.weight"] = np.zeros(3, dtype=np.float32)
    broken["model.layers.0.self_attn.q_proj.bias"] = np.zeros(7, dtype=np.float32)
    folder = str(tmp_path / "broken")
    plain.write_model_folder(folder, cfg, broken, store="F32")
    with pytest.raises(CppEngineError) as e:
        CppEngine(folder, dtype="float32", block_size=32, num_gpu_blocks=8, max_num_seqs=2, max_model_len=128, max_num_batched_tokens=64)
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.1.mlp.up_proj.weight" in msg and "lm_head.weight" in msg
    assert "unexpected tensors (1)" in msg and "model.layers.9.extra.weight" in msg and "wrong shapes (1)" in msg
    good = str(tmp_path / "good")
    plain.write_model_folder(good, cfg, w, store="F32")
    with pytest.raises(CppEngineError, match="Unknown model architecture"):
        CppEngine(good, model_arch="llama", dtype="float32", block_size=32, num_gpu_blocks=8, max_num_seqs=2, max_model_len=128)
    with pytest.raises(CppEngineError, match="block_size"):
        CppEngine(good, dtype="float32", block_size=24, num_gpu_blocks=8, max_num_seqs=2, max_model_len=128)
    with pytest.raises(CppEngineError, match="dtype"):
        CppEngine(good, dtype="float16", block_size=32, num_gpu_blocks=8, max_num_seqs=2, max_model_len=128)
    bad_cfg = str(tmp_path / "bad_cfg")
    plain.write_model_folder(bad_cfg, dict(cfg, num_attention_heads=5), w, store="F32")
    with pytest.raises(CppEngineError, match="multiple of"):
        CppEngine(bad_cfg, dtype="float32", block_size=32, num_gpu_blocks=8, max_num_seqs=2, max_model_len=128)
    # pages derived from the memory budget: never more than every request at full length needs
    eng = CppEngine(good, dtype="bfloat16", block_size=32, num_gpu_blocks=0, max_num_seqs=4, max_model_len=512, max_num_batched_tokens=64)
    assert eng.num_total_blocks == 4 * 16


def test_command_line(tmp_path):
    """vllm_cli with MODEL_PATH and MODEL_ARCH from the environment, flags overriding them."""
    from vllm_cpp_b200.csrc import build
    cfg, weights, folder, eng = cpp_engine(tmp_path, "A", "float32", seed=21, num_gpu_blocks=64)
    prompts = [token_ids(cfg, n, 50 + n) for n in (5, 17)]
    want = eng.generate(prompts, max_tokens=6, temperature=0.0, ignore_eos=True)
    eng.close()
    cli = build.build_engine()["cli"]
    env = dict(os.environ, MODEL_PATH=folder, MODEL_ARCH="qwen")
    args = [cli, "--dtype", "float32", "--num-blocks", "64", "--max-model-len", "256", "--max-num-batched-tokens", "256",
            "--max-tokens", "6", "--ignore-eos"]
    for p in prompts:
        args += ["--prompt-ids", ",".join(map(str, p))]
    out = subprocess.run(args, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert [[int(t) for t in line.split(",")] for line in out.stdout.strip().splitlines()] == want
    bad = subprocess.run([cli, "--model", str(tmp_path / "nowhere"), "--prompt-ids", "1"], capture_output=True, text=True, timeout=300)
    assert bad.returncode == 1 and "Cannot open config" in bad.stderr
    # random weights from a seed: a folder with config.json alone
    import json
    from vllm_cpp_b200.engine.cpp_host import CppEngine
    bare = tmp_path / "bare"
    bare.mkdir()
    (bare / "config.json").write_text(json.dumps(cfg))
    eng = CppEngine(str(bare), dtype="float32", num_gpu_blocks=64, max_model_len=256, max_num_batched_tokens=256,
                    load_format="random", seed=3)
    want = eng.generate(prompts, max_tokens=6, temperature=0.0, ignore_eos=True)
    eng.close()
    out = subprocess.run([cli, "--model", str(bare), "--load-format", "random", "--seed", "3"] + args[1:], env=env,
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert [[int(t) for t in line.split(",")] for line in out.stdout.strip().splitlines()] == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_weights_are_those_of_the_python_host(tmp_path, dtype):
    """load_format "random": the C++ host fills its weights from the seed with the same generator as
    write_random_model, so a folder written for that seed and a C++ engine that is given only config.json
    hold the same numbers: equal logits to the bit in float32 (the same kernels on the same values), and in
    bfloat16 as close as two runs of the same engine on the same weights."""
    import json
    from vllm_cpp_b200.engine.cpp_host import CppEngine
    from vllm_cpp_b200.weights.random_init import write_random_model
    cfg, page = CONFIGS["B"]
    cfg = dict(cfg, initializer_range=0.05)
    written = str(tmp_path / "written")
    write_random_model(written, cfg, seed=5, dtype=dtype)
    bare = tmp_path / "bare"
    bare.mkdir()
    (bare / "config.json").write_text(json.dumps(cfg))
    args = dict(dtype=dtype, block_size=page, num_gpu_blocks=24, max_num_seqs=4, max_model_len=256, max_num_batched_tokens=256)
    ids = token_ids(cfg, 70, 9)
    got = {}
    for name, folder, extra in (("loaded", written, {}), ("random", str(bare), dict(load_format="random", seed=5)),
                                ("other seed", str(bare), dict(load_format="random", seed=6))):
        eng = CppEngine(folder, **args, **extra)
        got[name] = eng.step_tokens([(0, ids[:50], [0, 49]), (1, ids[50:], [19])])
        eng.close()
    assert np.array_equal(got["loaded"], got["random"])
    assert np.abs(got["loaded"] - got["other seed"]).max() > 1e-3
    with pytest.raises(Exception, match="load_format"):
        CppEngine(str(bare), **args, load_format="gguf")


def test_both_hosts_give_the_same_tokens_under_pressure_in_float32(tmp_path):
    """150 requests on pages for six of them, 24 at a time, 200 tokens a step, a model of middling size with a
    windowed layer, an odd vocabulary of 32,003 and every sampling option (greedy, temperature, top-p, top-k,
    repetition penalty): in float32 the two hosts run the same kernels on the same numbers under the same
    scheduling decisions, so every request must get the same tokens from both, preempted or not.  (A last-bit
    difference in one host's rotation divisors was enough to part them here.)"""
    from vllm_cpp_b200 import EngineConfig, SamplingParams
    from vllm_cpp_b200.engine.cpp_host import CppEngine
    from vllm_cpp_b200.engine.llm_engine import Engine
    from vllm_cpp_b200.weights.random_init import write_random_model
    cfg = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 3, "vocab_size": 32003,
           "rope_theta": 1000000.0, "tie_word_embeddings": True, "use_sliding_window": True, "sliding_window": 96,
           "max_window_layers": 1, "max_position_embeddings": 4096, "hidden_act": "silu", "initializer_range": 0.05,
           "hidden_size": 520, "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 64,
           "intermediate_size": 1400, "rms_norm_eps": 1e-6}
    folder = str(tmp_path / "model")
    write_random_model(folder, cfg, seed=4, dtype="float32", device="cuda")
    n_req = 150
    rng = np.random.default_rng(8)
    lens, gens = rng.integers(4, 500, size=n_req), rng.integers(2, 90, size=n_req)
    prompts = [rng.integers(0, cfg["vocab_size"], size=int(n)).tolist() for n in lens]

    def options(i):
        return dict(max_tokens=int(gens[i]), temperature=0.9 if i % 3 else 0.0, top_p=0.85 if i % 5 == 0 else 1.0,
                    top_k=40 if i % 7 == 0 else -1, repetition_penalty=1.3 if i % 4 == 0 else 1.0, seed=77 + i, ignore_eos=True)

    common = dict(dtype="float32", block_size=16, num_gpu_blocks=240, max_num_seqs=24, max_model_len=640,
                  max_num_batched_tokens=200, max_tokens_per_step=200)
    eng = Engine(EngineConfig(model_path=folder, **common))
    ids = [eng.add_request(p, SamplingParams(**options(i))) for i, p in enumerate(prompts)]
    outs = {i: [] for i in ids}
    while eng.has_pending_work():
        for o in eng.step():
            outs[o.seq_id].extend(o.tokens)
    from_python = [outs[i] for i in ids]
    assert eng.scheduler.num_preemptions > 10 and eng.cache.num_free_pages() == 240
    del eng
    cpp = CppEngine(folder, **common)
    from_cpp = cpp.generate(prompts, per_request=[options(i) for i in range(n_req)])
    assert cpp.num_preemptions > 10 and cpp.num_free_blocks == 240
    cpp.close()
    assert [len(t) for t in from_python] == [int(g) for g in gens]
    differ = [i for i in range(n_req) if from_python[i] != from_cpp[i]]
    assert not differ, differ


@pytest.mark.parametrize("host", ["python", "cpp"])
@pytest.mark.parametrize("name,window,dtype", [("C", 24, "float32"), ("E", 70, "bfloat16"), ("D", 40, "bfloat16")])
def test_a_request_far_longer_than_the_pool_lives_on_its_window(tmp_path, name, window, dtype, host):
    """Every layer windowed: 700 tokens (portions, then one by one, decode steps captured on the Python host) on
    a pool of the window's pages and a few more, less than half of what the context would need; pages the window has
    passed are given back and used again.  Logits against the plain implementation at every position."""
    from helpers import Replayer
    from vllm_cpp_b200 import EngineConfig
    from vllm_cpp_b200.engine import factory
    from vllm_cpp_b200.engine.cpp_host import CppEngine
    page = CONFIGS[name][1]
    cfg = dict(CONFIGS[name][0], use_sliding_window=True, sliding_window=window, max_window_layers=0, max_position_embeddings=2048)
    weights = make_weights(cfg, 3, dtype)
    folder = model_folder(tmp_path, cfg, weights, dtype)
    n = 700
    ids = token_ids(cfg, n, 5)
    pages = -(-window // page) + 6
    assert pages * page * 2 < n
    if host == "python":
        model, cache, runner = factory.build(EngineConfig(model_path=folder, dtype=dtype, block_size=page, num_gpu_blocks=pages,
                                                          max_num_seqs=2, max_model_len=2048, max_num_batched_tokens=64,
                                                          use_cuda_graphs=True))
        rp, free = Replayer(runner, cache), (lambda: cache.num_free_pages())
    else:
        eng = CppEngine(folder, dtype=dtype, block_size=page, num_gpu_blocks=pages, max_num_seqs=2, max_model_len=2048,
                        max_num_batched_tokens=64)
        rp, free = CppReplayer(eng), (lambda: eng.num_free_blocks)
    at = 0
    for c in (40, 2, 17, 33):
        rp.step([("r", ids[at:at + c], range(c))])
        at += c
    while at < n:
        rp.step([("r", ids[at:at + 1], [0])])
        at += 1
    compare(rp.logits_of("r", range(n)), plain.forward(weights, cfg, ids), dtype, f"{name} {dtype} {host}")
    rp.step([("x", [1, 2], [])], end=["r", "x"])
    assert free() == pages
