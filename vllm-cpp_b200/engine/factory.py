"""Builds the model, its cache and the step function from an EngineConfig.

This is the reference's ``Engine::initialize`` + ``QwenModel::load_weights``
(src/core/engine.cpp:25-81, src/model/qwen.cpp:25-289) without the tokenizer:
read config.json, resolve the architecture in the registry, build the model from
its parts, load or generate the weights, size the cache, create the runner.  The
generation engine and the replay tool both start here.
"""
from __future__ import annotations

import sys
from typing import Tuple

import torch

from ..cache.manager import CacheManager, cdiv
from ..config.engine_config import ConfigError, EngineConfig
from ..config.registry import read_config_json, resolve_architecture
from ..parts.model import TORCH_DTYPES, DecoderModel, build_model as build_from_spec
from ..weights.loader import load_checkpoint
from ..weights.random_init import init_random_on_device
from .memory_plan import plan_for_model
from .runner import ModelRunner


def require_gpu() -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: this engine runs on a B200 (sm_100a) only; there is no CPU path")
    major, minor = torch.cuda.get_device_capability(0)
    if major != 10:
        print(f"[vllm_cpp_b200] warning: device has compute capability {major}.{minor}; "
              "the kernels are built for sm_100a only", file=sys.stderr)
    return torch.device("cuda", 0)


def build_model(cfg: EngineConfig, device) -> DecoderModel:
    if cfg.model_config is not None:
        config_json = cfg.model_config
    else:
        if not cfg.model_path:
            raise ConfigError("model_path is empty")
        config_json = read_config_json(cfg.model_path)
    typed, spec = resolve_architecture(config_json, cfg.model_arch)
    model = build_from_spec(spec, TORCH_DTYPES[cfg.dtype], device)
    model.typed_config = typed
    if cfg.load_format == "random":
        init_random_on_device(model, cfg.seed)
    else:
        load_checkpoint(model, cfg.model_path)
    return model


def build(cfg: EngineConfig) -> Tuple[DecoderModel, CacheManager, ModelRunner]:
    """Model, cache manager and runner for ``cfg`` on cuda:0."""
    device = require_gpu()
    # Library products keep float accumulation all the way; the float32 path does
    # not use them at all.
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_tf32 = False
    with torch.cuda.device(device), torch.no_grad():
        model = build_model(cfg, device)
        # the decode images of the weights may take a third of what the weights left free
        torch.cuda.empty_cache()
        free, total = torch.cuda.mem_get_info(device)
        usable = int(total * cfg.gpu_memory_utilization / 100) - (total - free)
        model.prepare_products(tune=cfg.tune_products, image_budget=max(0, usable // 3))
        max_model_len = min(cfg.max_model_len, model.spec.max_position_embeddings)
        # Every slice besides the pages is counted (engine/memory_plan.py); the workspace is allocated at the
        # size the plan gives it.  With an explicit num_gpu_blocks the plan only sizes the workspace.
        torch.cuda.synchronize()
        torch.cuda.empty_cache()                  # what loading left cached goes back, so that "free" is exact
        free, total = torch.cuda.mem_get_info(device)
        from ..csrc import ops
        try:
            planned = plan_for_model(cfg, model, total, total - free, max_model_len, ops.sm_count())
        except ConfigError:
            if cfg.num_gpu_blocks is None:
                raise
            planned = None
        specs = model.cache_specs()
        if cfg.num_gpu_blocks is not None:
            num_pages = cfg.num_gpu_blocks
        else:
            num_pages = planned.num_pages
            print("[vllm_cpp_b200] " + planned.table().replace("\n", "\n[vllm_cpp_b200] "), file=sys.stderr, flush=True)
        cache = CacheManager(specs, cfg.block_size, int(num_pages), cfg.max_num_seqs, model.dtype, device)
        runner = ModelRunner(model, cache, cfg.max_num_batched_tokens, cfg.max_num_seqs, max_model_len,
                             device, use_cuda_graphs=cfg.use_cuda_graphs,
                             workspace_bytes=planned.workspace_bytes if planned is not None else 0)
        runner.memory_plan = planned
    return model, cache, runner
