"""Where the device's memory goes: every slice the engine takes, counted before the cache is sized.

The reference makes one ``cudaMalloc`` and hands out slices of it
(include/vllm/memory/gpu_pool.hpp:12-41); the cache gets what an estimate of the other slices leaves
of ``free x gpu_memory_utilization`` (src/model/qwen.cpp:56-104).  Here torch's allocator owns the
memory, and the slices are counted exactly instead of estimated: the weights and their tile images
(measured, they are in place when the plan is made), the step's workspace at its high-water mark for
``max_num_batched_tokens`` tokens (the parts say what they take, and the workspace is allocated at
that size, so it never grows), the logits, the step's metadata, the sampler's buffers, the scratch
of the split kernels, the state slots, and a fixed reserve for what the libraries take on their own
(cuBLAS workspaces, the CUDA context's growth).  The rest of the budget is pages.

``plan`` is arithmetic on numbers and runs without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from ..cache.manager import CacheManager, cdiv
from ..config.engine_config import ConfigError, EngineConfig
from ..parts.base import StateSpec

LIBRARY_RESERVE = 384 << 20       # cuBLAS and cuBLASLt workspaces, graph pools, growth of the CUDA context
SAMPLER_SLOTS = 2                 # sampling.sampler.Sampler.SLOTS


def _round(n: int, to: int = 512) -> int:
    """torch's allocator hands out multiples of 512 bytes."""
    return (n + to - 1) // to * to


@dataclass
class MemoryPlan:
    rows: List[Tuple[str, int]] = field(default_factory=list)      # (slice, bytes), in the order they are taken
    budget: int = 0                # bytes this engine may hold in all: total x utilisation
    in_place: int = 0              # bytes already held on the device when the plan was made (weights, images, context)
    bytes_per_page: int = 0
    num_pages: int = 0
    workspace_bytes: int = 0
    pages_wanted: int = 0          # what every request at full length would need

    def table(self) -> str:
        lines = [f"memory plan: budget {self.budget / 2**30:.2f} GiB, {self.in_place / 2**30:.2f} GiB in place"]
        for name, n in self.rows:
            lines.append(f"  {name:<44s} {n / 2**20:12.1f} MiB")
        lines.append(f"  {'pages: ' + str(self.num_pages) + ' x ' + str(self.bytes_per_page) + ' B':<44s} "
                     f"{self.num_pages * self.bytes_per_page / 2**20:12.1f} MiB")
        return "\n".join(lines)


# Captured decode steps: at most this many are kept (the least recently replayed goes first), and each is
# counted at this many bytes per launch it holds (measured: 64 graphs of a 4-layer model took 10-18 MiB).
MAX_CAPTURED_STEPS = 256
CAPTURED_BYTES_PER_LAUNCH = 8 * 1024


def step_slices(cfg: EngineConfig, hidden: int, vocab: int, el: int, workspace_bytes: int, n_paged_groups: int,
                max_heads: int, max_head_dim: int, sm_count: int, state_bytes_per_slot: int,
                launches_per_step: int = 0) -> List[Tuple[str, int]]:
    """The slices besides weights and pages, for a model of these sizes: (name, bytes)."""
    n, r = cfg.max_num_batched_tokens, cfg.max_num_seqs
    max_blocks = cdiv(cfg.max_model_len, cfg.block_size)
    align = lambda x: (x + 3) // 4 * 4
    meta_ints = 3 * align(n) + align(r + 1) + 2 * align(r) + align(n) + n_paged_groups * align(r * max_blocks) + 64 * 1024
    rows = [
        ("step workspace (high-water mark)", _round(workspace_bytes)),
        ("logits [max_num_seqs, vocab] float32", _round(max(1, r) * vocab * 4)),
        ("step metadata (ids, positions, block tables)", _round(meta_ints * 4)),
        ("sampler options and ids, two steps in flight", SAMPLER_SLOTS * 3 * _round(4 * r * 4)),
        ("top-k/top-p scratch [max_num_seqs, vocab]", _round(r * vocab * 4)),
        ("product scratch (partial tiles, tickets)", _round(sm_count * 2 * 256 * 128 * 4) + _round(16384 * 4)),
        ("decode attention scratch (split merge)", _round(r * max_heads * 32 * (max_head_dim + 2) * 4) + _round(max(1024, r * max_heads) * 4)),
        ("state slots", _round(r * state_bytes_per_slot) if state_bytes_per_slot else 0),
        (f"captured decode steps (up to {MAX_CAPTURED_STEPS})",
         _round(MAX_CAPTURED_STEPS * launches_per_step * CAPTURED_BYTES_PER_LAUNCH) if cfg.use_cuda_graphs else 0),
        ("reserve for libraries and context", LIBRARY_RESERVE),
    ]
    return [(name, b) for name, b in rows if b]


def plan(cfg: EngineConfig, total: int, in_place: int, slices: List[Tuple[str, int]], bytes_per_page: int,
         max_model_len: int, already: Optional[List[Tuple[str, int]]] = None) -> MemoryPlan:
    """The page count that the budget leaves.  ``total``: the device's memory; ``in_place``: bytes the device
    already holds (everything, whoever holds it); ``slices``: what is still to be taken besides pages;
    ``already``: rows that only explain ``in_place`` (weights, images) in the printed table."""
    p = MemoryPlan(budget=int(total * cfg.gpu_memory_utilization / 100), in_place=in_place, bytes_per_page=max(1, bytes_per_page))
    p.rows = [(f"(in place) {name}", b) for name, b in (already or [])] + list(slices)
    p.workspace_bytes = next((b for name, b in slices if name.startswith("step workspace")), 0)
    left = p.budget - in_place - sum(b for _, b in slices)
    p.pages_wanted = cdiv(max_model_len, cfg.block_size) * cfg.max_num_seqs
    p.num_pages = max(0, min(p.pages_wanted, left // p.bytes_per_page))
    need = cdiv(max_model_len, cfg.block_size)
    if p.num_pages < need:
        raise ConfigError(
            f"not enough device memory for one request of max_model_len {max_model_len}: {p.num_pages} pages fit, "
            f"{need} are needed\n{p.table()}")
    return p


def plan_for_model(cfg: EngineConfig, model, total: int, in_place: int, max_model_len: int, sm_count: int) -> MemoryPlan:
    """``plan`` with the slices of ``model`` (a parts.model.DecoderModel whose weights are loaded)."""
    specs = model.cache_specs()
    el = torch.empty((), dtype=model.dtype).element_size()
    workspace = model.workspace_bytes(cfg.max_num_batched_tokens, cfg.max_num_seqs, cfg.max_num_seqs)
    state = sum(int(torch.empty((), dtype=s.dtype).element_size()) * int(torch.Size(s.shape).numel())
                for s in specs if isinstance(s, StateSpec))
    heads = [(getattr(p, "nh", 0), getattr(p, "d", 0)) for blk in model.blocks for p in blk.parts.values()]
    slices = step_slices(cfg, model.hidden, model.vocab, el, workspace, len({s for s in specs if hasattr(s, "num_kv_heads")}),
                         max((h for h, _ in heads), default=0), max((d for _, d in heads), default=0), sm_count, state,
                         launches_per_step=8 * len(model.spec.run_order) + 4)
    weights = sum(t.numel() * t.element_size() for t in model.tensors())
    images = sum(t.numel() * t.element_size() for t in model.tile_images())
    return plan(cfg, total, in_place, slices, CacheManager.bytes_per_page(specs, cfg.block_size, model.dtype), max_model_len,
                already=[("weights", weights), ("tile images of the weights", images)])
