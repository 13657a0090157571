#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen2.5-7B layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line.  ``value`` is decoded tokens per second at batch 8 with
contexts ending at 4,096 tokens, timed on the device with CUDA events around K
decode steps of the engine's step function (random bfloat16 weights, random token
ids, synthetic cache contents).  ``e2e`` is the same through the Python entry
point's engine: every step copies its inputs from pinned host memory to the
device and reads the sampled token ids back.  ``prefill`` times one 2,048-token
prompt in one step; ``points`` holds decode at batch 1 and 64; ``roofline`` sets
the decode step's bytes (every weight once, plus the cache of the live requests)
against the memory bandwidth.  A decode step reads about 15 GB, far more than the
126 MB of L2, so consecutive steps cannot serve each other from cache.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN25_7B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 3584, "num_hidden_layers": 28,
    "num_attention_heads": 28, "num_key_value_heads": 4, "intermediate_size": 18944, "vocab_size": 152064,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "use_sliding_window": False,
    "max_position_embeddings": 32768, "hidden_act": "silu", "initializer_range": 0.02,
}
# further sizes of the same architecture, for --size (layers, hidden, heads, kv heads, intermediate, rms eps)
SIZES = {
    "7b": dict(num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
               intermediate_size=18944, rms_norm_eps=1e-6),
    "14b": dict(num_hidden_layers=48, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                intermediate_size=13824, rms_norm_eps=1e-5),
    "32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                intermediate_size=27648, rms_norm_eps=1e-6),
}
CONTEXT = 4096
PREFILL_TOKENS = 2048
METRIC = "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Qwen2.5-7B bf16)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            hbm = float(p.get("hbm_gbs"))
            tf = float(p.get("bf16_tflops_sustained") or p.get("bf16_tflops"))
            return {"hbm_gbs": hbm, "bf16_tflops": tf, "source": "measured"}
        except (ValueError, TypeError, json.JSONDecodeError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                mhz.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(mhz)}


def write_timeline(path, batch, runner, cache, rng, vocab):
    """Kernel start and end times of one steady decode step, from the profiler's device-side records.
    Under programmatic dependent launch a kernel starts (its CTAs become resident) long before the
    kernel before it ends, so the column to read is how much later than its predecessor it ENDS."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    from vllm_cpp_b200.engine.runner import StepEntry
    ids = [f"t{i}" for i in range(batch)]
    for r in ids:
        cache.add_request(r)
        cache.reserve(r, CONTEXT - 64)
        cache.commit(r, CONTEXT - 64)

    def one():
        runner.step([StepEntry(r, [int(rng.integers(0, vocab))], [0]) for r in ids])

    for _ in range(4):
        one()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(2):
            one()
        torch.cuda.synchronize()
    tmp = path + ".trace.json"
    prof.export_chrome_trace(tmp)
    with open(tmp) as f:
        ev = [e for e in json.load(f)["traceEvents"] if e.get("cat") == "kernel"]
    os.remove(tmp)
    for r in ids:
        cache.free_request(r)
    ev.sort(key=lambda e: e["ts"])
    ev = ev[len(ev) // 2:]                          # the second step
    t0 = ev[0]["ts"]
    rows = sorted(((e["ts"] + e["dur"] - t0, e["ts"] - t0, e["name"]) for e in ev))
    with open(path, "w") as f:
        f.write(f"# one decode step, batch {batch}, contexts {CONTEXT - 60}: end, start (us from the step's first kernel), "
                "end minus previous end, kernel\n")
        prev = 0.0
        for end, start, name in rows:
            f.write(f"{end:9.2f} {start:9.2f} {end - prev:8.2f}  {name[:90]}\n")
            prev = end


def run_mix(cfg, a) -> int:
    """Continuous batching through the engine's own API: requests of mixed lengths arrive at once, prompts
    are read in portions of at most 2,048 tokens a step beside the tokens other requests decode."""
    import numpy as np
    import torch
    from vllm_cpp_b200 import EngineConfig, SamplingParams
    from vllm_cpp_b200.engine.llm_engine import Engine
    n_req, gen, budget = 32, 256, 2048
    rng = np.random.default_rng(3)
    lens = rng.integers(128, 4097, size=n_req)
    pages = int(sum(-(-(int(n) + gen) // 16) for n in lens)) + 64
    ecfg = EngineConfig(load_format="random", model_config=cfg, seed=0, dtype="bfloat16", block_size=16,
                        num_gpu_blocks=pages, max_num_seqs=n_req, max_model_len=4096 + gen,
                        max_num_batched_tokens=budget, max_tokens_per_step=budget)
    engine = Engine(ecfg)
    sp = SamplingParams(max_tokens=gen, temperature=0.0, ignore_eos=True)

    def run():
        for n in lens:
            engine.add_request(rng.integers(0, cfg["vocab_size"], size=int(n)).tolist(), sp)
        torch.cuda.synchronize()
        t, steps, out = time.perf_counter(), 0, 0
        while engine.has_pending_work():
            out += len(engine.step())
            steps += 1
        torch.cuda.synchronize()
        return time.perf_counter() - t, steps, out

    run()                                             # warm-up: sizes workspaces, captures graphs
    dt, steps, out = run()
    prompt = int(lens.sum())
    print(json.dumps({"metric": "continuous batching: 32 requests, prompts 128-4096, 256 generated each, 2048 tokens a step",
                      "value": round(out / dt, 1), "unit": "generated tokens/s", "seconds": round(dt, 3), "steps": steps,
                      "prompt_tokens": prompt, "generated_tokens": out,
                      "all_tokens_per_s": round((prompt + out) / dt, 1), "preemptions": engine.scheduler.num_preemptions,
                      "config": {"model": f"Qwen2.5-{a.size.upper()} layer sizes", "layers": cfg["num_hidden_layers"]}}))
    return 0


def model_numbers(cfg):
    h, nh, nkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = h // nh
    inter, v, layers = cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    per_layer = (nh + 2 * nkv) * d * h + nh * d * h + 3 * inter * h
    return {"layer_params": per_layer, "matrix_params": layers * per_layer + v * h,
            "kv_bytes_per_token": layers * 2 * nkv * d * 2, "d": d}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=QWEN25_7B["num_hidden_layers"],
                    help="fewer layers than the 28 of the configuration (recorded in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--size", default="7b", choices=sorted(SIZES),
                    help="layer sizes: Qwen2.5-7B (the benchmark's), 14B or 32B")
    ap.add_argument("--mix", action="store_true",
                    help="instead of the fixed-batch measurement: 32 requests with prompts of 128 to 4,096 tokens and "
                         "256 generated tokens each through the engine, 2,048 tokens a step (continuous batching)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="run one part only (for profiling); the other fields of the line are null")
    ap.add_argument("--no-pdl", action="store_true", help="ordinary launches instead of programmatic dependent launch")
    ap.add_argument("--library-gemm", action="store_true", help="cuBLAS for every bfloat16 product (no tcgen05 kernel)")
    ap.add_argument("--timeline", metavar="FILE", default=None,
                    help="with --only decode: also write the device timeline of one decode step (every kernel's "
                         "start and end as CUPTI reports them through torch.profiler) to FILE as text")
    ap.add_argument("--no-cuda-graphs", action="store_true",
                    help="launch every kernel of a decode step directly (for a profiler's launch list)")
    a = ap.parse_args()
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "jiamumuzhao/vllm-cpp is a CMake C++ project with no setup.py or pyproject.toml, so the "
                          "offline pip install refuses it; its engine also forwards one token per call and "
                          "overwrites the embedding with an untied lm_head, so it cannot run this 7B workload"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py measures one GPU (N=1); this engine has no multi-GPU path, --gpus {a.gpus} is not run")
        return 2
    steps, warmup = max(1, a.steps), max(3, a.warmup)

    import torch
    from vllm_cpp_b200 import EngineConfig, SamplingParams
    from vllm_cpp_b200.csrc import ops
    from vllm_cpp_b200.engine.llm_engine import Engine
    from vllm_cpp_b200.engine.runner import StepEntry

    if a.no_pdl:
        ops.set_pdl(False)
    if a.library_gemm:
        ops.set_tcgen05_linear(False)
    cfg = dict(QWEN25_7B, **SIZES[a.size])
    if a.size == "7b" or a.layers != QWEN25_7B["num_hidden_layers"]:
        cfg["num_hidden_layers"] = a.layers
    if a.mix:
        return run_mix(cfg, a)
    nums = model_numbers(cfg)
    peaks = load_peaks()
    max_batch = max(64, a.batch)
    pages = max_batch * (CONTEXT // 16 + 2) + PREFILL_TOKENS // 16 + 16
    ecfg = EngineConfig(load_format="random", model_config=cfg, seed=0, dtype="bfloat16", block_size=16,
                        num_gpu_blocks=pages, max_num_seqs=max_batch, max_model_len=CONTEXT + 16,
                        max_num_batched_tokens=PREFILL_TOKENS, max_tokens_per_step=PREFILL_TOKENS,
                        use_cuda_graphs=not a.no_cuda_graphs)
    t0 = time.time()
    engine = Engine(ecfg)
    runner, cache = engine.runner, engine.cache
    torch.cuda.synchronize()
    load_s = time.time() - t0
    gen = torch.Generator(device="cuda").manual_seed(1)
    for g in cache.paged:                       # synthetic cache contents for the decode runs
        g.pages.normal_(0.0, 0.5, generator=gen)
    vocab = cfg["vocab_size"]
    rng = __import__("numpy").random.default_rng(0)

    def time_decode(batch, n_steps, n_warm):
        """Device time of n_steps decode steps at ``batch`` requests whose contexts end at CONTEXT."""
        start_ctx = CONTEXT - n_steps - n_warm
        ids = [f"d{batch}_{i}" for i in range(batch)]
        for r in ids:
            cache.add_request(r)
            cache.reserve(r, start_ctx)
            cache.commit(r, start_ctx)
        toks = rng.integers(0, vocab, size=(n_steps + n_warm, batch))
        temperature = torch.zeros(batch, device="cuda")
        uniform = torch.zeros(batch, device="cuda")
        out = torch.empty(batch, dtype=torch.int32, device="cuda")

        def one(k):
            logits = runner.step([StepEntry(r, [int(toks[k, i])], [0]) for i, r in enumerate(ids)])
            ops.sample(logits, temperature, uniform, out)

        for k in range(n_warm):
            one(k)
        torch.cuda.synchronize()
        launches0 = ops.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.nvtx.range_push("timed_decode")
        e0.record()
        for k in range(n_warm, n_warm + n_steps):
            one(k)
        e1.record()
        torch.cuda.synchronize()
        torch.cuda.nvtx.range_pop()
        ms = e0.elapsed_time(e1) / n_steps
        launches = ops.launch_count() - launches0
        kv_bytes = batch * (CONTEXT - n_steps / 2) * nums["kv_bytes_per_token"]
        for r in ids:
            cache.free_request(r)
        return ms, launches, kv_bytes

    def time_prefill(reps, n_warm):
        times = []
        for k in range(reps + n_warm):
            cache.add_request("p")
            toks = rng.integers(0, vocab, size=PREFILL_TOKENS).tolist()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if k >= n_warm:
                torch.cuda.nvtx.range_push("timed_prefill")
            e0.record()
            runner.step([StepEntry("p", toks, [PREFILL_TOKENS - 1])])
            e1.record()
            torch.cuda.synchronize()
            if k >= n_warm:
                torch.cuda.nvtx.range_pop()
            cache.free_request("p")
            if k >= n_warm:
                times.append(e0.elapsed_time(e1))
        return statistics.median(times)

    def time_e2e(batch, n_steps, n_warm):
        """Wall time of engine.step() in steady decode: pinned inputs in, sampled ids out, every step.
        Prompts are fed first (in portions, some requests already decoding beside them); the timed
        steps start when every request decodes, and end before the first one finishes."""
        portions = -(-CONTEXT // PREFILL_TOKENS)
        slack = batch * portions + 2
        n_warm = max(n_warm, 64)        # the prompts' steps leave reduced clocks behind: decode until they are back
        budget = n_steps + n_warm + slack
        prompt_len = CONTEXT - budget
        sp = SamplingParams(max_tokens=budget, temperature=0.0, ignore_eos=True)
        ids = [engine.add_request(rng.integers(0, vocab, size=prompt_len).tolist(), sp) for _ in range(batch)]
        seqs = [engine.sequences[i] for i in ids]
        while engine.scheduler.waiting or any(s.remaining > 1 or s.output_len == 0 for s in seqs):
            engine.step()
        for _ in range(n_warm):
            engine.step()
        assert all(s.output_len + n_steps <= budget for s in seqs) and len(engine.scheduler.running) == batch
        torch.cuda.synchronize()
        t = time.perf_counter()
        produced = 0
        for _ in range(n_steps):
            produced += len(engine.step())
        torch.cuda.synchronize()
        dt = time.perf_counter() - t
        assert produced == batch * n_steps
        h2d = int(runner.last_meta_bytes) + 4 * 4 * batch        # step metadata + four floats of sampling options a row
        for i in ids:
            engine.abort_request(i)
        return produced / dt, h2d, 4 * batch

    if a.only == "prefill":
        ms = time_prefill(max(1, min(steps, 3)), 2)
        print(json.dumps({"metric": METRIC, "only": "prefill", "prefill_ms": round(ms, 3),
                          "value": round(PREFILL_TOKENS / (ms * 1e-3), 1), "unit": "tokens/s"}))
        return 0
    clocks = ClockSampler()
    clocks.start()
    ms, launches, kv_bytes = time_decode(a.batch, steps, warmup)
    clock_info = clocks.stop()
    if a.only == "decode" and a.timeline:
        write_timeline(a.timeline, a.batch, runner, cache, rng, vocab)
    if a.only == "decode":
        print(json.dumps({"metric": METRIC, "only": "decode", "batch": a.batch, "ms_per_step": round(ms, 4),
                          "value": round(a.batch / (ms * 1e-3), 1), "unit": "tokens/s", "gpu_launches": launches,
                          "cuda_graphs": not a.no_cuda_graphs, "clocks": clock_info}))
        return 0

    weight_bytes = nums["matrix_params"] * 2
    step_bytes = weight_bytes + kv_bytes
    achieved = step_bytes / (ms * 1e-3) / 1e9
    value = a.batch / (ms * 1e-3)

    # The decode figures first, the prefill last: the prefill steps run at the power limit, and what is
    # measured right after them runs at the reduced clocks they leave behind for a while (batch 1 read
    # 3.15-3.26 ms a step after them against 3.08 ms before).
    points = {}
    if not a.skip_points:
        for b in (1, 64):
            pms, _, _ = time_decode(b, max(8, steps // 2), 3)
            points[f"decode_b{b}"] = round(b / (pms * 1e-3), 1)
    e2e_value, h2d, d2h = time_e2e(a.batch, steps, warmup)

    prefill_ms = time_prefill(3, 2)
    t = PREFILL_TOKENS
    flops = 2.0 * (nums["matrix_params"] - vocab * cfg["hidden_size"]) * t + 2.0 * vocab * cfg["hidden_size"] \
        + cfg["num_hidden_layers"] * 4.0 * cfg["num_attention_heads"] * nums["d"] * (t * (t + 1) / 2)
    prefill = {"value": round(t / (prefill_ms * 1e-3), 1), "tokens": t, "ms": round(prefill_ms, 3),
               "frac": round(flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4),
               "tflops": round(flops / (prefill_ms * 1e-3) / 1e12, 1)}

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": {"model": f"Qwen2.5-{a.size.upper()} layer sizes", "layers": cfg["num_hidden_layers"],
                   "layers_of_configuration": SIZES[a.size]["num_hidden_layers"], "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": nums["d"], "intermediate": cfg["intermediate_size"], "vocab": vocab,
                   "global_batch": a.batch, "seq_len": CONTEXT, "kv_block": 16, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (a decode step reads %.1f GB)" % (step_bytes / 1e9),
                   "cuda_graphs": bool(ecfg.use_cuda_graphs), "overlap_steps": bool(ecfg.overlap_decode_steps),
                   "peaks": peaks["source"], "load_s": round(load_s, 1)},
        "clocks": clock_info,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
