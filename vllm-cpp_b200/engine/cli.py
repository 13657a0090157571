"""Command line in the manner of the reference's ``src/main.cpp``.

The reference's program takes ``--model``, ``--arch``, ``--port`` and
``--quantization`` (src/main.cpp:26-37) and its launcher script turns the
environment variables MODEL_PATH, MODEL_ARCH, QUANT_MODE and PORT into those
flags (scripts/run_server.sh:7-10,41-46); then it serves HTTP.  This program takes
the same ``--model`` and ``--arch`` (and the same environment variables as
defaults), refuses a quantization other than none, has no server and so no port,
and generates from token ids given on the command line or in a file.

    python -m vllm_cpp_b200.engine.cli --model DIR --prompt-ids 1,2,3 --max-tokens 16
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams


def parse_args(argv=None):
    d = EngineConfig()
    ap = argparse.ArgumentParser(prog="vllm_cpp_b200", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default=os.environ.get("MODEL_PATH", "./models/test-model"),
                    help="model folder (config.json, model.safetensors); default $MODEL_PATH")
    ap.add_argument("--arch", default=os.environ.get("MODEL_ARCH", ""),
                    help="architecture name, e.g. qwen; default $MODEL_ARCH, else config.json's architectures[0]")
    ap.add_argument("--quantization", default=os.environ.get("QUANT_MODE", "none"),
                    help="only 'none': quantized weights are not built")
    ap.add_argument("--dtype", default=d.dtype, choices=["bfloat16", "float32"])
    ap.add_argument("--load-format", default=d.load_format, choices=["safetensors", "random"])
    ap.add_argument("--seed", type=int, default=d.seed)
    ap.add_argument("--block-size", type=int, default=d.block_size)
    ap.add_argument("--num-gpu-blocks", type=int, default=None)
    ap.add_argument("--gpu-memory-utilization", type=int, default=d.gpu_memory_utilization)
    ap.add_argument("--max-num-seqs", type=int, default=d.max_num_seqs)
    ap.add_argument("--max-model-len", type=int, default=d.max_model_len)
    ap.add_argument("--max-num-batched-tokens", type=int, default=d.max_num_batched_tokens)
    ap.add_argument("--max-tokens-per-step", type=int, default=d.max_tokens_per_step)
    ap.add_argument("--prompt-ids", action="append", default=[],
                    help="comma-separated token ids of one prompt; may be given several times")
    ap.add_argument("--prompt-file", help="JSON file: a list of lists of token ids")
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=d.temperature)
    ap.add_argument("--top-p", type=float, default=d.top_p)
    ap.add_argument("--top-k", type=int, default=d.top_k)
    ap.add_argument("--repetition-penalty", type=float, default=d.repetition_penalty)
    ap.add_argument("--sample-seed", type=int, default=None)
    ap.add_argument("--no-tuning", action="store_true",
                    help="do not measure product kernels and grids at load: the same tokens from every run")
    ap.add_argument("--ignore-eos", action="store_true")
    return ap.parse_args(argv)


def main(argv=None) -> int:
    a = parse_args(argv)
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in a.prompt_ids]
    if a.prompt_file:
        with open(a.prompt_file) as f:
            prompts += json.load(f)
    if not prompts:
        print("no prompt given (--prompt-ids or --prompt-file)", file=sys.stderr)
        return 2
    from .llm import LLM
    print(f"vllm_cpp_b200 starting\nModel: {a.model} Arch: {a.arch or '(from config.json)'}", file=sys.stderr)
    t0 = time.time()
    llm = LLM(a.model, model_arch=a.arch, quant_mode=a.quantization, dtype=a.dtype, load_format=a.load_format,
              seed=a.seed, block_size=a.block_size, num_gpu_blocks=a.num_gpu_blocks,
              gpu_memory_utilization=a.gpu_memory_utilization, max_num_seqs=a.max_num_seqs,
              max_model_len=a.max_model_len, max_num_batched_tokens=a.max_num_batched_tokens,
              max_tokens_per_step=a.max_tokens_per_step, tune_products=not a.no_tuning)
    t1 = time.time()
    sp = SamplingParams(max_tokens=a.max_tokens, temperature=a.temperature, top_p=a.top_p, top_k=a.top_k,
                        repetition_penalty=a.repetition_penalty, seed=a.sample_seed, ignore_eos=a.ignore_eos)
    outs = llm.generate(prompts, sp)
    t2 = time.time()
    for o in outs:
        print(",".join(str(t) for t in o))
    n = sum(len(o) for o in outs)
    print(f"loaded in {t1 - t0:.2f}s; generated {n} tokens in {t2 - t1:.3f}s ({n / max(t2 - t1, 1e-9):.1f} tok/s)",
          file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
