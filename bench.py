#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen2.5-7B layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line.  ``value`` is decoded tokens per second at batch 8 while the contexts grow
from 2,048 to 4,096 tokens: the K timed steps are taken in up to four runs of consecutive steps
placed evenly along that growth (the first run starts at 2,048 tokens, the last ends at 4,096), on
the device with CUDA events around the engine's step function (random bfloat16 weights, random
token ids, synthetic cache contents); ``points`` holds the two ends and the same mean at batch 1
and 64.  ``e2e`` is the same through the Python entry point's engine: requests with prompts of
2,048 tokens generate up to 4,096, every step copies its inputs from pinned host memory to the
device and reads the sampled token ids back, and the same runs of steps are timed by the wall
clock.  ``prefill`` times one 2,048-token prompt in one step; ``roofline`` sets the decode steps'
bytes (every weight once, plus the cache of the live requests) against the memory bandwidth.  A
decode step reads about 15 GB, far more than the 126 MB of L2, so consecutive steps cannot serve
each other from cache.

``--impl reference`` runs the unmodified jiamumuzhao/vllm-cpp (built by baseline/build_reference.py
into baseline/_ref) on the same configuration and the same runs of steps, through its own model
interface as its engine drives it: one forward per token and sequence (baseline/ref_driver.cpp).
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
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
CONTEXT_START = 2048          # the contexts of the decode measurement grow from here ...
CONTEXT = 4096                # ... to here
SLACK = 64                    # room beyond CONTEXT: requests that began a few steps earlier than others pass it
PREFILL_TOKENS = 2048
METRIC = "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Qwen2.5-7B bf16)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            burst = float(p.get("bf16_tflops"))
            return {"hbm_gbs": float(p.get("hbm_gbs")), "bf16_tflops": burst,
                    "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained") or burst), "source": "measured"}
        except (ValueError, TypeError, json.JSONDecodeError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


def decode_runs(steps: int):
    """[(context at the run's first step, steps)]: ``steps`` timed decode steps in up to four runs of
    consecutive steps placed evenly along the growth of the contexts from CONTEXT_START to CONTEXT; the
    last run ends with the contexts at CONTEXT."""
    n = 4 if steps >= 8 else 2 if steps >= 2 else 1
    sizes = [steps // n + (1 if i < steps % n else 0) for i in range(n)]
    if n == 1:
        return [(CONTEXT - sizes[0], sizes[0])]
    last = CONTEXT - sizes[-1]
    return [(CONTEXT_START + round(i * (last - CONTEXT_START) / (n - 1)), k) for i, k in enumerate(sizes)]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the measurements run; ``mark`` names the
    stretch of time that follows, so that every sample can be laid to the measurement it fell into."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.proc = None
        self.marks = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def mark(self, name):
        self.marks.append((time.time(), name))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.mark(None)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        by_region, mx, reasons = {}, None, {}
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                stamp = time.mktime(time.strptime(f[0][:19], "%Y/%m/%d %H:%M:%S")) + float("0" + f[0][19:])
                mhz, mx = float(f[1]), float(f[2])
            except ValueError:
                continue
            region = None
            for t, name in self.marks:
                if stamp >= t:
                    region = name
            if region is None:
                continue
            by_region.setdefault(region, []).append(mhz)
            for n, v in zip(self.NAMES, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.setdefault(region, set()).add(n)
        decode = [m for r, v in by_region.items() if r != "prefill" for m in v]
        info = {"sm_mhz": statistics.median(decode) if decode else None, "sm_max_mhz": mx,
                "reasons": sorted(set().union(*[v for r, v in reasons.items() if r != "prefill"])) if reasons else [],
                "samples": len(decode)}
        if by_region.get("prefill"):
            info["prefill_sm_mhz"] = statistics.median(by_region["prefill"])
            info["prefill_reasons"] = sorted(reasons.get("prefill", ()))
        return info


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
    are read in portions of at most 2,048 tokens a step beside the tokens other requests decode.  Also
    prints where a step's time goes (the engine's per-phase timers)."""
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
                        max_num_batched_tokens=budget, max_tokens_per_step=budget, time_phases=True)
    engine = Engine(ecfg)
    sp = SamplingParams(max_tokens=gen, temperature=0.0, ignore_eos=True)

    def run():
        for n in lens:
            engine.add_request(rng.integers(0, cfg["vocab_size"], size=int(n)).tolist(), sp)
        torch.cuda.synchronize()
        t, steps, out = time.perf_counter(), 0, 0
        phases = {}
        while engine.has_pending_work():
            out += len(engine.step())
            steps += 1
            for k, v in engine.last_stats.phase_ms.items():
                phases[k] = phases.get(k, 0.0) + v
        torch.cuda.synchronize()
        return time.perf_counter() - t, steps, out, phases

    run()                                             # warm-up: sizes workspaces, captures graphs
    dt, steps, out, phases = run()
    prompt = int(lens.sum())
    print(json.dumps({"metric": "continuous batching: 32 requests, prompts 128-4096, 256 generated each, 2048 tokens a step",
                      "value": round(out / dt, 1), "unit": "generated tokens/s", "seconds": round(dt, 3), "steps": steps,
                      "prompt_tokens": prompt, "generated_tokens": out,
                      "all_tokens_per_s": round((prompt + out) / dt, 1), "preemptions": engine.scheduler.num_preemptions,
                      "phase_ms_per_step": {k: round(v / steps, 4) for k, v in sorted(phases.items())},
                      "config": {"model": f"Qwen2.5-{a.size.upper()} layer sizes", "layers": cfg["num_hidden_layers"]}}))
    return 0


def model_numbers(cfg):
    h, nh, nkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = h // nh
    inter, v, layers = cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    per_layer = (nh + 2 * nkv) * d * h + nh * d * h + 3 * inter * h
    return {"layer_params": per_layer, "matrix_params": layers * per_layer + v * h,
            "kv_bytes_per_token": layers * 2 * nkv * d * 2, "d": d}


def flat_config(cfg, a, nums, extra):
    out = {"model": f"Qwen2.5-{a.size.upper()} layer sizes", "layers": cfg["num_hidden_layers"],
           "layers_of_configuration": SIZES[a.size]["num_hidden_layers"], "hidden": cfg["hidden_size"],
           "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": nums["d"],
           "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": a.batch,
           "seq_len": CONTEXT, "decode_contexts": f"{CONTEXT_START} growing to {CONTEXT}", "kv_block": 16,
           "parallelism": "single GPU"}
    out.update(extra)
    return out


# ------------------------------------------------------------------------------------------- the C++ host
def run_cpp_host(cfg, a) -> int:
    """Decode throughput through the C++ host runtime (vllm::Engine behind include/vllm/vllm.hpp): the same random
    weights, requests with prompts of 2,048 tokens generating up to 4,096, the same runs of timed steps as the
    e2e figure of the Python host, by the wall clock around Engine::step (which returns the sampled ids)."""
    import numpy as np
    from vllm_cpp_b200.engine.cpp_host import CppEngine
    folder = tempfile.mkdtemp(prefix="vcb_cpp_model_")          # config.json alone: the weights come from the seed
    try:
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg, f)
        batch, lead = a.batch, 16
        pages = batch * ((CONTEXT + SLACK) // 16 + 1) + 16
        t0 = time.time()
        eng = CppEngine(folder, dtype="bfloat16", block_size=16, num_gpu_blocks=pages, max_num_seqs=max(batch, 8),
                        max_model_len=CONTEXT + SLACK, max_num_batched_tokens=PREFILL_TOKENS, max_tokens_per_step=PREFILL_TOKENS,
                        fused_decode_tokens=int(os.environ.get("VCB_FUSED_DECODE_TOKENS", "64")), load_format="random", seed=0)
        load_s = time.time() - t0
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    rng = np.random.default_rng(0)
    prompt_len = CONTEXT_START - lead
    for _ in range(batch):
        eng.add_request(rng.integers(0, cfg["vocab_size"], size=prompt_len).tolist(), max_tokens=CONTEXT + SLACK - prompt_len,
                        temperature=0.0, ignore_eos=True)
    produced = [0] * batch
    def step():
        outs = eng.step()
        for rid, _, _ in outs:
            produced[rid] += 1
        return len(outs)
    while min(produced) == 0 or len(set(produced)) > 1 and max(produced) < 2:      # until every request decodes
        step()
    runs, timed, seconds = decode_runs(max(1, a.steps)), 0, 0.0
    for ctx0, k in runs:
        while prompt_len + min(produced) < ctx0:
            step()
        t = time.perf_counter()
        got = sum(step() for _ in range(k))
        seconds += time.perf_counter() - t
        assert got == batch * k, (got, batch, k)
        timed += k
    print(json.dumps({"host": "cpp", "metric": METRIC, "value": round(batch * timed / seconds, 1), "unit": "tokens/s",
                      "ms_per_step": round(seconds / timed * 1e3, 4), "steps": timed, "batch": batch,
                      "config": {"model": f"Qwen2.5-{a.size.upper()} layer sizes", "layers": cfg["num_hidden_layers"],
                                 "decode_contexts": f"{CONTEXT_START} growing to {CONTEXT}", "load_s": round(load_s, 1),
                                 "pool_gb": round(eng.pool_total_bytes / 1e9, 2)}}))
    return 0


# ---------------------------------------------------------------------------------------- kernels one by one
def run_kernels(cfg) -> int:
    """Every kernel of the step alone at the benchmark's layer sizes: microseconds (CUDA events around a CUDA
    graph of several launches on rotating buffers, so that neither the host nor the L2 cache flatters them) and
    what that is in GB/s of the bytes the kernel must move or in TFLOP/s.  One text table."""
    import numpy as np
    import torch
    from vllm_cpp_b200.csrc import ops
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    h, nh, nkv, inter, vocab = (cfg[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads",
                                                 "intermediate_size", "vocab_size"))
    d, page, bf = h // nh, 16, torch.bfloat16
    dev = "cuda"
    rows = []

    def rnd(*shape, dtype=bf, scale=1.0):
        return (torch.randn(*shape, device=dev) * scale).to(dtype)

    def add(name, fn, n_copies, bytes_=0, flops=0):
        us = ops.time_in_graph(fn, reps=max(4, n_copies))
        rows.append((name, us, bytes_ / us / 1e3 if bytes_ else None, flops / us / 1e6 if flops else None))

    for t in (8, 2048):
        copies = 6 if t == 8 else 3
        ids = torch.randint(0, vocab, (t,), dtype=torch.int32, device=dev)
        table = rnd(vocab, h, scale=0.02)
        res = [torch.zeros(t, h, device=dev) for _ in range(copies)]
        add(f"embedding, {t} tokens", lambda i: ops.embedding(table, ids, res[i % copies]), copies, bytes_=t * h * 6)
        delta, normed = [rnd(t, h) for _ in range(copies)], [torch.empty(t, h, dtype=bf, device=dev) for _ in range(copies)]
        gain = torch.ones(h, device=dev)
        add(f"residual add + RMSNorm, {t} tokens",
            lambda i: ops.add_rmsnorm(res[i % copies], delta[i % copies], gain, normed[i % copies], 1e-6), copies, bytes_=t * h * 12)
        del table
        # bias + rotation + cache write
        width = (nh + 2 * nkv) * d
        qkv, q_out = [rnd(t, width) for _ in range(copies)], torch.empty(t, nh * d, dtype=bf, device=dev)
        cache = torch.zeros(t // page + 2, 2, nkv, page * d, dtype=bf, device=dev)
        pos = torch.arange(t, dtype=torch.int32, device=dev)
        req = torch.zeros(t, dtype=torch.int32, device=dev)
        bt = torch.arange(t // page + 2, dtype=torch.int32, device=dev).view(1, -1)
        denom = torch.from_numpy(np.power(np.float32(1e6), np.arange(d // 2, dtype=np.float32) * 2 / d).astype(np.float32)).to(dev)
        bias = torch.zeros(width, device=dev)
        add(f"q/k/v bias + rotation + cache write, {t} tokens",
            lambda i: ops.rope_cache_write(qkv[i % copies], bias, pos, req, bt, denom, q_out, cache, num_heads=nh, num_kv_heads=nkv,
                                           head_dim=d, rotary_dim=d, pairing=0, page_size=page, write_kv=True),
            copies, bytes_=t * width * 4)
    # SwiGLU on the library's gate-and-up product (prefill)
    t = 2048
    gu, act = [rnd(t, 2 * inter) for _ in range(2)], torch.empty(t, inter, dtype=bf, device=dev)
    add("silu(gate) * up, 2,048 tokens", lambda i: ops.silu_mul(gu[i % 2], act), 2, bytes_=t * inter * 6)
    del gu, act
    # products: the engine's kernel at 8 tokens (plain epilogue; the fused ones are in the decode timeline), the library's at 2,048
    shapes = [("qkv", (nh + 2 * nkv) * d, h), ("output projection", h, nh * d), ("gate and up", 2 * inter, h), ("down", h, inter)]
    for name, n, k in shapes:
        copies = 6 if n * k < 1e8 else 3
        ws = [rnd(n, k, scale=0.02) for _ in range(copies)]
        for w in ws:
            ops.tile_weights(w)
        x8, o8 = rnd(8, k), torch.empty(8, n, dtype=bf, device=dev)
        add(f"product {name} [{n} x {k}], 8 tokens (tcgen05)", lambda i: ops.gemm_bf16_tcgen05(x8, ws[i % copies], o8), copies,
            bytes_=n * k * 2)
        x, o = rnd(2048, k), torch.empty(2048, n, dtype=bf, device=dev)
        add(f"product {name}, 2,048 tokens (cuBLAS)", lambda i: ops._library_mm(x, ws[i % copies], o), copies, flops=2.0 * 2048 * n * k)
        del ws
    head = rnd(vocab, h, scale=0.02)
    ops.tile_weights(head)
    x8, logits = rnd(8, h), torch.empty(8, vocab, device=dev)
    add(f"output product [{vocab} x {h}], 8 rows, float32 logits", lambda i: ops.gemm_bf16_tcgen05(x8, head, logits), 4, bytes_=vocab * h * 2)
    del head
    # attention
    for t in (2048, 8192):
        n_pages = t // page + 2
        cache = rnd(n_pages, 2, nkv, page * d, scale=0.5)
        q, out = rnd(t, nh * d), torch.empty(t, nh * d, dtype=bf, device=dev)
        bt = torch.arange(n_pages, dtype=torch.int32, device=dev).view(1, -1)
        q_start = torch.tensor([0, t], dtype=torch.int32, device=dev)
        ctx = torch.zeros(1, dtype=torch.int32, device=dev)
        g = nh // nkv
        n_tiles = -(-t * g // ops.TC_ATTENTION_TILE_ROWS)
        order = np.argsort(-np.arange(n_tiles), kind="stable")          # the tiles with the most keys first
        tile_req = torch.zeros(n_tiles, dtype=torch.int32, device=dev)
        tile_row0 = torch.from_numpy((np.arange(n_tiles, dtype=np.int32) * ops.TC_ATTENTION_TILE_ROWS)[order].copy()).to(dev)
        add(f"prefill attention, one prompt of {t}", lambda i: ops.attention_prefill_tc(
            q, cache, out, q_start, ctx, bt, tile_req, tile_row0, num_heads=nh, num_kv_heads=nkv, head_dim=d, page_size=page,
            window=0, scale=d ** -0.5), 4, flops=4.0 * nh * d * t * (t + 1) / 2)
    from vllm_cpp_b200.config.model_spec import PartSpec
    from vllm_cpp_b200.engine.runner import HostStep
    from vllm_cpp_b200.parts.attention import PagedAttention
    part = PagedAttention(h, nh, nkv, d, True, False, 0, PartSpec("none"), bf, dev)
    mixed = [128 + round(i * (4352 - 128) / 31) for i in range(32)]
    for batch, contexts, label in ((8, [CONTEXT - 1] * 8, f"contexts of {CONTEXT}"), (64, [CONTEXT - 1] * 64, f"contexts of {CONTEXT}"),
                                   (32, mixed, "contexts of 128 to 4,352")):
        blocks = -(-(max(contexts) + 1) // page)
        cache = rnd(batch * blocks + 1, 2, nkv, page * d, scale=0.5)
        q, out = rnd(batch, nh * d), torch.empty(batch, nh * d, dtype=bf, device=dev)
        bt = torch.arange(batch * blocks, dtype=torch.int32, device=dev).view(batch, blocks)
        q_start = torch.arange(batch + 1, dtype=torch.int32, device=dev)
        ctx = torch.tensor(contexts, dtype=torch.int32, device=dev)
        host = HostStep([1] * batch, list(contexts), page)
        split_tiles = torch.from_numpy(part.step_arrays()[part._splits_key()](host)).to(dev)
        nsplit = host.shapes[part._splits_key()]
        need = batch * nh * nsplit
        po, pml = torch.empty(need * d, device=dev), torch.empty(need * 2, device=dev)
        tickets = torch.zeros(batch * nkv, dtype=torch.int32, device=dev)
        add(f"decode attention, batch {batch}, {label}", lambda i: ops.attention_decode_mma(
            q, cache, out, q_start, ctx, bt, None, batch, nsplit, po, pml, tickets, num_heads=nh, num_kv_heads=nkv, head_dim=d,
            page_size=page, window=0, scale=d ** -0.5, split_tiles=split_tiles), 4,
            bytes_=sum(c + 1 for c in contexts) * 2 * nkv * d * 2)
        del cache
    logits = rnd(64, vocab, dtype=torch.float32)
    temp, uni, ids = torch.zeros(64, device=dev), torch.zeros(64, device=dev), torch.empty(64, dtype=torch.int32, device=dev)
    add("sampling (greedy), 64 rows", lambda i: ops.sample(logits, temp, uni, ids), 4, bytes_=64 * vocab * 4)
    temp.fill_(0.8)
    add("sampling (temperature), 64 rows", lambda i: ops.sample(logits, temp, uni, ids), 4, bytes_=64 * vocab * 4)
    w = torch.empty(2 * inter, h, dtype=bf, device=dev)
    add("random weights, one gate-and-up matrix", lambda i: ops.random_normal(w, 12345 + i, 0.0, 0.02), 4, bytes_=w.numel() * 2)
    ops.check_status()
    peaks = load_peaks()
    print(f"# kernels alone, Qwen2.5-7B layer sizes, bfloat16; peaks ({peaks['source']}): {peaks['hbm_gbs']:.0f} GB/s, "
          f"{peaks['bf16_tflops']:.0f} TFLOP/s (burst)")
    print(f"{'kernel':<62s} {'us':>9s} {'GB/s':>8s} {'TFLOP/s':>8s} {'of peak':>8s}")
    for name, us, gbs, tf in rows:
        frac = gbs / peaks["hbm_gbs"] if gbs else tf / peaks["bf16_tflops"]
        print(f"{name:<62s} {us:9.1f} {gbs if gbs else float('nan'):8.0f} {tf if tf else float('nan'):8.1f} {frac:8.2f}")
    return 0


# ------------------------------------------------------------------------------------------ reference arm
REFERENCE_NOTES = ("the reference's own faults at these sizes, none of which changes the work of a step: an untied lm_head is "
                   "copied over the embedding table (src/model/qwen.cpp:279-281); the bias area of 3*1024 floats a layer "
                   "(qwen.cpp:67,113-114,179-181) is overrun by 7B's 4,608 and the surplus lands, inside the same pool, on "
                   "layer 0's rotation table below position 336")


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:600]}))
    return 0


def run_reference(cfg, a) -> int:
    """The reference's own speed on the same configuration: write the model folder, run baseline/_ref/ref_driver."""
    if a.gpus != 1:
        return unavailable("jiamumuzhao/vllm-cpp has no multi-GPU path")
    try:
        from baseline.build_reference import driver_env, driver_path
        driver = driver_path()
    except Exception as e:                                # the build's own message is the reason
        return unavailable(f"the reference could not be built here: {e}")
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        from vllm_cpp_b200.weights.random_init import write_random_model
    except Exception as e:
        return unavailable(f"cannot prepare the model folder: {e}")
    nums = model_numbers(cfg)
    params = nums["matrix_params"] + cfg["vocab_size"] * cfg["hidden_size"]          # with the embedding table
    need_file = params * 2 + (64 << 20)
    # the reference's loader keeps every tensor as host float32 (src/model/model_loader.cpp:61,100) beside the file
    need_ram = params * 4 + need_file + (8 << 30)
    with open("/proc/meminfo") as f:
        avail = next(int(l.split()[1]) * 1024 for l in f if l.startswith("MemAvailable"))
    where = next((d for d in ("/dev/shm", tempfile.gettempdir()) if os.path.isdir(d)
                  and shutil.disk_usage(d).free > need_file + (4 << 30)), None)
    if where is None:
        return unavailable(f"no room for the {need_file >> 30} GB model folder in /dev/shm or the temporary folder")
    if avail < need_ram:
        return unavailable(f"the reference's loader needs about {need_ram >> 30} GB of host memory "
                           f"(float32 copies of all tensors), {avail >> 30} GB are available")
    runs = decode_runs(max(1, a.steps))
    per_run = min(k for _, k in runs)
    runs = [(c, per_run) for c, _ in runs]                # the driver takes one length for all runs
    warm = max(3, a.warmup)
    folder = tempfile.mkdtemp(prefix="vcb_ref_model_", dir=where)
    try:
        t0 = time.time()
        write_random_model(folder, cfg, seed=0, dtype="bfloat16", device="cuda")
        torch.cuda.empty_cache()
        write_s = time.time() - t0
        print(f"[bench] model folder written in {write_s:.0f} s", file=sys.stderr, flush=True)
        # batch 64 is left out unless asked for: one forward of the reference at these contexts takes a
        # good part of a second, and a step of 64 sequences is 64 of them
        batches = [a.batch] + ([] if a.skip_points else [b for b in ((1, 64) if a.reference_b64 else (1,)) if b != a.batch])
        cmd = [driver, "bench", "--model", folder, "--batches", ",".join(map(str, batches)),
               "--contexts", ",".join(str(c) for c, _ in runs), "--steps-per-context", str(per_run),
               "--warmup", str(warm), "--prefill", str(PREFILL_TOKENS), "--max-model-len", str(CONTEXT + 16),
               "--block-size", "16", "--budget-s", str(a.reference_budget_s)]
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=None, text=True, env=driver_env())
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    lines = [l for l in p.stdout.strip().splitlines() if l.startswith("{")]
    if p.returncode != 0 or not lines:
        tail = p.stdout.strip().splitlines()[-3:]
        return unavailable(f"the reference's run ended with code {p.returncode}: {' | '.join(tail)}")
    res = json.loads(lines[-1])
    if "error" in res:
        return unavailable(f"the reference's run stopped: {res['error']}")
    by_batch = {r["batch"]: r["decode"] for r in res["runs"]}
    main = by_batch[a.batch]
    steps = per_run * len(main)
    ms = sum(d["device_ms_per_step"] for d in main) / len(main)
    e2e_ms = sum(d["e2e_ms_per_step"] for d in main) / len(main)
    points = {f"decode_b{a.batch}_ctx{main[0]['context']}": round(a.batch / (main[0]["device_ms_per_step"] * 1e-3), 2),
              f"decode_b{a.batch}_ctx{main[-1]['context'] + per_run}": round(a.batch / (main[-1]["device_ms_per_step"] * 1e-3), 2)}
    for b, dec in by_batch.items():
        if b != a.batch:
            points[f"decode_b{b}"] = round(b / (sum(d["device_ms_per_step"] for d in dec) / len(dec) * 1e-3), 2)
    blocks = res["blocks_per_seq"]
    line = {
        "impl": "reference", "metric": METRIC, "value": round(a.batch / (ms * 1e-3), 2), "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": warm, "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp16 operands, fp32 accumulation, activations and cache (the reference's only mode)",
        "data": "synthetic: the same random weights N(0,0.02) as the other arm, written as a bfloat16 model folder; random token ids",
        "config": flat_config(cfg, a, nums, {
            "how": "QwenModel::forward, one call per token and sequence, as Engine::decode and Engine::prefill call it",
            "cache": "zeros as the reference's pool is cleared to, plus what the steps write",
            "load_s": res["load_s"], "write_model_s": round(write_s, 1), "notes": REFERENCE_NOTES}),
        "e2e": {"value": round(a.batch / (e2e_ms * 1e-3), 2), "unit": "tokens/s",
                # per sequence: the token id, and per layer the block table and the context length; the logits back
                "h2d_bytes_per_step": a.batch * (4 + res["layers"] * 4 * (blocks + 1)),
                "d2h_bytes_per_step": a.batch * 4 * res["vocab"]},
        "gpu_launches": None,
        "prefill": ({"value": round(res["prefill"]["tokens"] / (res["prefill"]["ms"] * 1e-3), 1), "tokens": res["prefill"]["tokens"],
                     "ms": round(res["prefill"]["ms"], 1), "how": "one forward per token",
                     # a prompt cut short by the time budget is not the 2,048-token prompt of the metric
                     "same_config": res["prefill"]["tokens"] == PREFILL_TOKENS} if res["prefill"]["tokens"] else None),
        "points": points, "seconds": res["seconds"],
    }
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------------------------ our arm
def main() -> int:
    global CONTEXT_START, CONTEXT, PREFILL_TOKENS, SLACK
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
    ap.add_argument("--kernels", action="store_true",
                    help="instead of the step: every kernel alone at these layer sizes, a text table of microseconds "
                         "and achieved GB/s or TFLOP/s")
    ap.add_argument("--host", default="python", choices=["python", "cpp"],
                    help="cpp: decode throughput through the C++ host runtime (vllm::Engine) instead of the Python host")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--prefill-tokens", type=int, default=0,
                    help=f"with --only prefill: tokens of the one prompt instead of {PREFILL_TOKENS}")
    ap.add_argument("--contexts", default="",
                    help="START,END: the decode measurement's contexts grow from START to END tokens instead of "
                         f"{CONTEXT_START},{CONTEXT} (with --only decode; the default is the benchmark's configuration)")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="run one part only (for profiling); the other fields of the line are null")
    ap.add_argument("--no-pdl", action="store_true", help="ordinary launches instead of programmatic dependent launch")
    ap.add_argument("--library-gemm", action="store_true", help="cuBLAS for every bfloat16 product (no tcgen05 kernel)")
    ap.add_argument("--timeline", metavar="FILE", default=None,
                    help="with --only decode: also write the device timeline of one decode step (every kernel's "
                         "start and end as CUPTI reports them through torch.profiler) to FILE as text")
    ap.add_argument("--no-cuda-graphs", action="store_true",
                    help="launch every kernel of a decode step directly (for a profiler's launch list)")
    ap.add_argument("--utilization", type=int, default=0, metavar="PERCENT",
                    help="let the engine size its own cache from this share of the device's memory "
                         "(gpu_memory_utilization) instead of a fixed number of pages")
    ap.add_argument("--reference-budget-s", type=float, default=1300.0,
                    help="--impl reference: begin no further measurement after this many seconds")
    ap.add_argument("--reference-b64", action="store_true", help="--impl reference: measure batch 64 too (many minutes)")
    a = ap.parse_args()
    if a.contexts:
        CONTEXT_START, CONTEXT = (int(v) for v in a.contexts.split(","))
        if a.only != "decode" or not 0 < CONTEXT_START < CONTEXT:
            ap.error("--contexts START,END goes with --only decode and needs 0 < START < END")
    if a.prefill_tokens:
        if a.only != "prefill" or a.prefill_tokens < 2:
            ap.error("--prefill-tokens N goes with --only prefill")
        PREFILL_TOKENS = a.prefill_tokens
        CONTEXT_START, CONTEXT = max(CONTEXT_START, PREFILL_TOKENS), max(CONTEXT, PREFILL_TOKENS + 64)
    SLACK = max(SLACK, a.batch + 32)          # requests begin a prompt's step apart: the first is a batch of steps ahead of the last
    cfg = dict(QWEN25_7B, **SIZES[a.size])
    if a.size == "7b" or a.layers != QWEN25_7B["num_hidden_layers"]:
        cfg["num_hidden_layers"] = a.layers
    if a.impl == "reference":
        return run_reference(cfg, a)
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
    if a.mix:
        return run_mix(cfg, a)
    if a.kernels:
        return run_kernels(cfg)
    if a.host == "cpp":
        return run_cpp_host(cfg, a)
    nums = model_numbers(cfg)
    peaks = load_peaks()
    max_batch = a.batch if a.only != "all" else max(64, a.batch)        # the points at batch 1 and 64 use the same engine
    pages = max_batch * ((CONTEXT + SLACK) // 16 + 1) + PREFILL_TOKENS // 16 + 16
    ecfg = EngineConfig(load_format="random", model_config=cfg, seed=0, dtype="bfloat16", block_size=16,
                        num_gpu_blocks=None if a.utilization else pages,
                        gpu_memory_utilization=a.utilization or 90, max_num_seqs=max_batch, max_model_len=CONTEXT + SLACK,
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
    runs = decode_runs(steps)

    def time_decode(batch, n_warm):
        """Device time of the timed runs of decode steps at ``batch`` requests: [(context, steps, ms)], launches."""
        temperature = torch.zeros(batch, device="cuda")
        uniform = torch.zeros(batch, device="cuda")
        out = torch.empty(batch, dtype=torch.int32, device="cuda")
        results, launches = [], 0
        for ctx0, k in runs:
            toks = rng.integers(0, vocab, size=(max(k, n_warm), batch))

            def requests(tag):                  # requests whose caches hold ctx0 tokens (synthetic contents)
                ids = [f"d{batch}_{ctx0}_{tag}{i}" for i in range(batch)]
                for r in ids:
                    cache.add_request(r)
                    cache.reserve(r, ctx0)
                    cache.commit(r, ctx0)
                return ids

            def one(ids, j):
                logits = runner.step([StepEntry(r, [int(toks[j, i])], [0]) for i, r in enumerate(ids)])
                ops.sample(logits, temperature, uniform, out)

            # warm-up: the run itself once over, with requests of its own, so that the timed steps find
            # their launch shapes captured (a step whose longest context enters a new power-of-two bucket,
            # as 2,048 -> 2,049 does, is otherwise launched directly once and captured once)
            ids = requests("w")
            for j in range(max(k, n_warm)):
                one(ids, j)
            for r in ids:
                cache.free_request(r)
            ids = requests("t")
            torch.cuda.synchronize()
            before = ops.launch_count()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.nvtx.range_push("timed_decode")
            e0.record()
            for j in range(k):
                one(ids, j)
            e1.record()
            torch.cuda.synchronize()
            torch.cuda.nvtx.range_pop()
            results.append((ctx0, k, e0.elapsed_time(e1)))
            launches += ops.launch_count() - before
            for r in ids:
                cache.free_request(r)
        return results, launches

    def summary(batch, results):
        """tokens/s over all runs, ms per step, bytes the steps had to read."""
        total_ms = sum(ms for _, _, ms in results)
        n = sum(k for _, k, _ in results)
        kv = sum(batch * (c + (k - 1) / 2 + 1) * nums["kv_bytes_per_token"] * k for c, k, _ in results)
        return batch * n / (total_ms * 1e-3), total_ms / n, nums["matrix_params"] * 2 * n + kv

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

    def time_e2e(batch):
        """Wall time of engine.step() over the same runs of steps: requests with prompts just short of
        CONTEXT_START tokens generate until their contexts reach CONTEXT; pinned inputs in, sampled ids out, every
        step.  A run is timed between two synchronisations; the steps between the runs are not timed."""
        lead = 64                               # steps before the first run: the prompts' steps leave reduced clocks behind
        prompt_len = CONTEXT_START - lead
        sp = SamplingParams(max_tokens=CONTEXT + SLACK - prompt_len, temperature=0.0, ignore_eos=True)
        ids = [engine.add_request(rng.integers(0, vocab, size=prompt_len).tolist(), sp) for _ in range(batch)]
        seqs = [engine.sequences[i] for i in ids]
        while engine.scheduler.waiting or any(s.remaining > 1 or s.output_len == 0 for s in seqs):
            engine.step()
        produced, seconds = 0, 0.0
        for ctx0, k in runs:
            while min(s.num_processed_tokens for s in seqs) < ctx0:
                engine.step()
            assert len(engine.scheduler.running) == batch
            torch.cuda.synchronize()
            t = time.perf_counter()
            got = 0
            for _ in range(k):
                got += len(engine.step())
            torch.cuda.synchronize()
            seconds += time.perf_counter() - t
            assert got == batch * k, (got, batch, k)
            produced += got
        h2d = int(runner.last_meta_bytes) + 4 * 4 * batch        # step metadata + four floats of sampling options a row
        for i in ids:
            engine.abort_request(i)
        return produced / seconds, h2d, 4 * batch

    def prefill_flops(t):
        """The products of every layer and the output product of the one wanted row, and causal attention."""
        return 2.0 * (nums["matrix_params"] - vocab * cfg["hidden_size"]) * t + 2.0 * vocab * cfg["hidden_size"] \
            + cfg["num_hidden_layers"] * 4.0 * cfg["num_attention_heads"] * nums["d"] * (t * (t + 1) / 2)

    if a.only == "prefill":
        ms = time_prefill(max(1, min(steps, 3)), 2)
        tf = prefill_flops(PREFILL_TOKENS) / (ms * 1e-3) / 1e12
        print(json.dumps({"metric": METRIC, "only": "prefill", "tokens": PREFILL_TOKENS, "prefill_ms": round(ms, 3),
                          "value": round(PREFILL_TOKENS / (ms * 1e-3), 1), "unit": "tokens/s", "tflops": round(tf, 1),
                          "frac": round(tf / peaks["bf16_tflops"], 4),
                          "frac_of_sustained_peak": round(tf / peaks["bf16_tflops_sustained"], 4)}))
        return 0
    clocks = ClockSampler()
    clocks.start()
    clocks.mark("decode")
    results, launches = time_decode(a.batch, warmup)
    value, ms, step_bytes = summary(a.batch, results)
    if a.only == "decode":
        clock_info = clocks.stop()
        if a.timeline:
            write_timeline(a.timeline, a.batch, runner, cache, rng, vocab)
        print(json.dumps({"metric": METRIC, "only": "decode", "batch": a.batch, "ms_per_step": round(ms, 4),
                          "value": round(value, 1), "unit": "tokens/s", "gpu_launches": launches,
                          "contexts": [CONTEXT_START, CONTEXT],
                          "roofline": {"achieved": round(step_bytes / (ms * sum(k for _, k, _ in results) * 1e-3) / 1e9, 1),
                                       "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                       "frac": round(step_bytes / (ms * sum(k for _, k, _ in results) * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)},
                          "runs": [[c, k, round(t / k, 4)] for c, k, t in results],
                          "product_grids": {f"{n}x{k} tile {bn}{' gated' if g else ''}{' residual' if r else ''}": c
                                            for (n, k, bn, g, r), c in sorted(ops._cta_choice.items())},
                          "layer_products_us": getattr(engine.model, "tuning_report", {}).get("layer_products_us"),
                          "cuda_graphs": not a.no_cuda_graphs, "clocks": clock_info}))
        return 0
    n_timed = sum(k for _, k, _ in results)
    achieved = step_bytes / (ms * n_timed * 1e-3) / 1e9

    # The decode figures first, the prefill last: the prefill steps run at the power limit, and what is
    # measured right after them runs at the reduced clocks they leave behind for a while.
    (c_first, k_first, t_first), (c_last, k_last, t_last) = results[0], results[-1]
    points = {f"decode_b{a.batch}_ctx{c_first}": round(a.batch * k_first / (t_first * 1e-3), 1),
              f"decode_b{a.batch}_ctx{c_last + k_last}": round(a.batch * k_last / (t_last * 1e-3), 1)}
    if not a.skip_points:
        for b in (1, 64):
            if b != a.batch:
                res_b, _ = time_decode(b, 3)
                points[f"decode_b{b}"] = round(summary(b, res_b)[0], 1)
    clocks.mark("e2e")
    e2e_value, h2d, d2h = time_e2e(a.batch)
    clocks.mark("prefill")
    prefill_ms = time_prefill(3, 2)
    clock_info = clocks.stop()
    t = PREFILL_TOKENS
    tflops = prefill_flops(t) / (prefill_ms * 1e-3) / 1e12
    prefill = {"value": round(t / (prefill_ms * 1e-3), 1), "tokens": t, "ms": round(prefill_ms, 3),
               # one step timed alone between synchronisations: the burst peak is its denominator
               "frac": round(tflops / peaks["bf16_tflops"], 4),
               "frac_of_sustained_peak": round(tflops / peaks["bf16_tflops_sustained"], 4), "tflops": round(tflops, 1)}

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": n_timed,
        "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": flat_config(cfg, a, nums, {
            "l2": "inputs larger than L2 (a decode step reads %.1f GB)" % (step_bytes / n_timed / 1e9),
            "cuda_graphs": bool(ecfg.use_cuda_graphs), "overlap_steps": bool(ecfg.overlap_decode_steps),
            "peaks": peaks["source"], "load_s": round(load_s, 1), "kv_pages": cache.num_pages}),
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
