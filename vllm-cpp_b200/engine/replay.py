"""Trace replay: feed given token ids through the model step by step, write logits.

It samples nothing and schedules nothing: every step of the trace is handed as it
is to ``ModelRunner.step``, the function that generation uses, on the same model,
cache manager and kernels.  The nearest thing in the reference is the recompute
replay after preemption (include/vllm/core/sequence.hpp:37-40,
src/core/engine.cpp:153-166), which also rebuilds state from given token ids.

Input, one JSON object per line on standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose
logits are wanted.  ``end``: requests that are finished after this step; their
pages and slot are given back.  For a step that wants something, the logits are
written to ``<out>/<step>.f32`` as little-endian float32 [wanted, vocab], in the
order of the entries and of ``want``.  After every step ``done <step>`` is printed
and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

from ..cache.manager import cdiv
from ..config.engine_config import EngineConfig
from .runner import StepEntry

MAX_LIVE_REQUESTS = 8


def replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int, lines, out=sys.stdout,
           block_size: int = 16, model_arch: str = "") -> int:
    from . import factory
    if max_tokens <= 0:
        raise ValueError("--max-tokens must be positive")
    os.makedirs(out_dir, exist_ok=True)
    pages = cdiv(max_tokens, block_size)
    cfg = EngineConfig(model_path=model_dir, model_arch=model_arch, dtype=dtype, block_size=block_size,
                       num_gpu_blocks=pages, max_num_seqs=MAX_LIVE_REQUESTS,
                       max_model_len=pages * block_size, max_num_batched_tokens=pages * block_size,
                       use_cuda_graphs=False)
    model, cache, runner = factory.build(cfg)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step_no = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            if e["id"] not in cache.requests:
                cache.add_request(e["id"])
            entries.append(StepEntry(e["id"], list(e["tokens"]), list(e.get("want", []))))
        if entries:
            logits = runner.step(entries)
            if logits.shape[0]:
                arr = logits.detach().cpu().numpy().astype("<f4", copy=False)
                tmp = os.path.join(out_dir, f".{step_no}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, f"{step_no}.f32"))
        for rid in rec.get("end", []):
            if rid in cache.requests:
                cache.free_request(rid)
        print(f"done {step_no}", file=out, flush=True)
    import torch
    torch.cuda.synchronize()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time; the cache pool is made for this many")
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--arch", default="", help="architecture name; default: config.json's architectures[0]")
    a = ap.parse_args(argv)
    return replay(a.model, a.dtype, a.out, a.max_tokens, sys.stdin, sys.stdout, a.block_size, a.arch)


if __name__ == "__main__":
    sys.exit(main())
