"""Per-request sampling options.

The reference's per-request options are ``max_tokens``, ``temperature``, ``top_p``
and ``top_k`` (include/vllm/core/engine.hpp:50-54; HTTP defaults
src/server/http_server.cpp:157-165) plus the engine-wide ``repetition_penalty``
(src/core/engine.cpp:214).  ``temperature <= 0`` means greedy
(src/sampler/sampler.cpp:38).  Added here: a seed, since the reference's generator
is seeded from random_device and cannot be reproduced (sampler.cpp:68), explicit
stop ids (the reference stops on the tokenizer's <|im_end|> / <|endoftext|>,
src/tokenizer/tokenizer.cpp:339-349), and ``ignore_eos`` for benchmarks.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class SamplingParams:
    max_tokens: int = 64
    temperature: Optional[float] = None        # None: the engine's default
    top_p: Optional[float] = None
    top_k: Optional[int] = None                # -1: off
    repetition_penalty: Optional[float] = None
    seed: Optional[int] = None                 # None: derived from the engine's seed and the request id
    stop_token_ids: Optional[List[int]] = None   # None: the model's eos ids
    ignore_eos: bool = False

    def resolved(self, engine_cfg, default_stop_ids) -> "SamplingParams":
        p = SamplingParams(
            max_tokens=self.max_tokens,
            temperature=engine_cfg.temperature if self.temperature is None else float(self.temperature),
            top_p=engine_cfg.top_p if self.top_p is None else float(self.top_p),
            top_k=engine_cfg.top_k if self.top_k is None else int(self.top_k),
            repetition_penalty=(engine_cfg.repetition_penalty if self.repetition_penalty is None
                                else float(self.repetition_penalty)),
            seed=self.seed,
            stop_token_ids=list(default_stop_ids) if self.stop_token_ids is None else list(self.stop_token_ids),
            ignore_eos=self.ignore_eos)
        if p.max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        if not (0.0 < p.top_p <= 1.0):
            raise ValueError(f"top_p must lie in (0, 1], got {p.top_p}")
        if not (p.top_k == -1 or p.top_k > 0):
            raise ValueError(f"top_k is -1 (off) or positive, got {p.top_k}")
        if not p.repetition_penalty > 0:
            raise ValueError("repetition_penalty must be positive")
        return p
