"""Typed engine configuration.

Field names and meanings follow the reference's ``EngineConfig``
(include/vllm/core/config.hpp:34-66): ``model_path``, ``model_arch``,
``gpu_memory_utilization`` (a percentage, 0-100), ``block_size`` (tokens per KV
page), ``max_num_seqs``, ``max_model_len``, ``max_num_batched_tokens``,
``max_tokens_per_step`` (the chunked-prefill budget) and the sampling defaults
``temperature``, ``top_p``, ``top_k``, ``repetition_penalty``.  The reference
validates only ``block_size``, ``gpu_memory_utilization`` and ``max_num_seqs``
(src/model/qwen.cpp:48-52); every field is validated here.

Fields the reference declares but never reads (``min_p``, ``frequency_penalty``,
``presence_penalty``, ``schedule_policy``, ``enable_prefix_caching``) and the
server's ``port`` have no effect in the reference and are not carried over.
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Optional

DTYPES = ("bfloat16", "float32")
LOAD_FORMATS = ("safetensors", "random")
QUANT_MODES = ("none",)


class ConfigError(ValueError):
    """A configuration value that the engine refuses, with the reason."""


@dataclass
class EngineConfig:
    # Model
    model_path: str = ""
    # "" means: take config.json's architectures[0].  The reference takes the
    # name only from --arch (src/core/engine.cpp:40).
    model_arch: str = ""
    # Precision of weights, activations and cache.  "float32" is a true 32-bit
    # path: no reduced-precision matrix mode anywhere.
    dtype: str = "bfloat16"
    quant_mode: str = "none"
    # "safetensors" reads model_path/model.safetensors; "random" builds weights
    # on the device from `seed` for the sizes in model_path/config.json (or in
    # `model_config`), without touching the disk.
    load_format: str = "safetensors"
    seed: int = 0
    # A dict with the architecture's config.json keys; used instead of
    # model_path/config.json when given (random weights only).
    model_config: Optional[dict] = None

    # Memory
    gpu_memory_utilization: int = 90      # percent of the device's memory
    block_size: int = 16                  # tokens per KV page
    # Pages per cache group.  None: derived from gpu_memory_utilization after
    # weights and work buffers are placed.
    num_gpu_blocks: Optional[int] = None
    max_num_seqs: int = 64
    max_model_len: int = 8192
    max_num_batched_tokens: int = 16384   # most tokens in one step

    # Scheduling
    max_tokens_per_step: int = 512        # most prompt tokens in one step
    # Where a preempted request re-enters the waiting queue.  The reference
    # pushes it to the back (src/core/scheduler.cpp:183).
    preempted_to_front: bool = False

    # Sampling defaults (per request values override them)
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    repetition_penalty: float = 1.0

    # Measure at load which product kernel and which grid are fastest for each shape on this device (bfloat16).
    # What is measured may come out differently by timing noise from one engine to the next on the same device;
    # sums are then taken in another order and a sampled token may differ in the last bit's favour.  False pins
    # every few-token product to the engine's own kernel on its default grid: the same tokens from every engine.
    tune_products: bool = True
    # Capture pure-decode steps in CUDA graphs.
    use_cuda_graphs: bool = True
    # While every running request decodes, launch the next step before this step's tokens
    # have reached the host (they are fed to it on the device), so the GPU never waits for
    # the host between steps.  The tokens are the same either way in float32; in bfloat16 too, unless a request
    # meets a stop token while the step after is already on its way: that step then runs with one request more
    # than it would have had, and a product over 17 rows does not round as one over 16.
    overlap_decode_steps: bool = True
    # Time the phases of every step (schedule, pack, launch, sample, wait on the host; forward and
    # sampling on the device with CUDA events) into StepStats.phase_ms.  The reference has a scoped
    # host timer for this (include/vllm/utils/profiler.hpp:15-53).
    time_phases: bool = False

    def __post_init__(self):
        self.validate()

    def validate(self) -> None:
        def need(cond, msg):
            if not cond:
                raise ConfigError(msg)

        need(self.dtype in DTYPES, f"dtype must be one of {DTYPES}, got {self.dtype!r}")
        need(self.quant_mode in QUANT_MODES,
             f"quant_mode {self.quant_mode!r}: quantized weights are not built; only 'none'")
        need(self.load_format in LOAD_FORMATS,
             f"load_format must be one of {LOAD_FORMATS}, got {self.load_format!r}")
        need(isinstance(self.block_size, int) and self.block_size > 0,
             "block_size must be a positive integer (KV block size must be greater than zero)")
        need(self.block_size % 16 == 0 and self.block_size <= 256,
             f"block_size must be a multiple of 16 and at most 256, got {self.block_size}")
        need(0 < self.gpu_memory_utilization <= 100,
             f"gpu_memory_utilization is a percentage in (0, 100], got {self.gpu_memory_utilization}")
        need(self.max_num_seqs > 0, "max_num_seqs must be positive")
        need(self.max_model_len > 0, "max_model_len must be positive")
        need(self.max_num_batched_tokens > 0, "max_num_batched_tokens must be positive")
        need(self.max_tokens_per_step > 0, "max_tokens_per_step must be positive")
        need(self.num_gpu_blocks is None or self.num_gpu_blocks > 0,
             "num_gpu_blocks must be positive when given")
        need(self.top_p > 0.0 and self.top_p <= 1.0, f"top_p must lie in (0, 1], got {self.top_p}")
        need(self.top_k == -1 or self.top_k > 0, f"top_k is -1 (off) or positive, got {self.top_k}")
        need(self.repetition_penalty > 0.0, "repetition_penalty must be positive")
        need(self.load_format == "random" or self.model_config is None,
             "model_config (an in-memory config.json) is only for load_format='random'")

    @classmethod
    def field_names(cls):
        return [f.name for f in fields(cls)]
