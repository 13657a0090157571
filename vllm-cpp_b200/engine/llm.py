"""The Python entry point: ``LLM(model_path, ...).generate(prompts, params)``.

The reference has no Python API; its users drive ``Engine::add_request`` and
``Engine::step`` from C++ (src/server/http_server.cpp:124-155).  ``LLM`` wraps
those two calls: all prompts are queued, the engine steps until every request is
finished, and the generated ids come back in the order of the prompts.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from .llm_engine import Engine


class LLM:
    def __init__(self, model: str = "", **engine_args):
        """``model``: a folder with config.json and model.safetensors.  ``engine_args``:
        fields of EngineConfig (dtype, block_size, max_num_seqs, load_format, ...)."""
        unknown = set(engine_args) - set(EngineConfig.field_names())
        if unknown:
            raise TypeError(f"unknown engine options {sorted(unknown)}; known: {EngineConfig.field_names()}")
        self.engine = Engine(EngineConfig(model_path=model, **engine_args))

    def generate(self, prompt_token_ids: Sequence[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None
                 ) -> List[List[int]]:
        """Generated token ids for each prompt (the stop token, if one ended it, included)."""
        n = len(prompt_token_ids)
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            params = [sampling_params] * n
        else:
            params = list(sampling_params)
            if len(params) != n:
                raise ValueError("one SamplingParams per prompt, or one for all")
        ids = [self.engine.add_request(p, sp) for p, sp in zip(prompt_token_ids, params)]
        results = {i: [] for i in ids}
        while self.engine.has_pending_work():
            outs = self.engine.step()
            if not outs and not self.engine.last_stats.num_tokens:
                raise RuntimeError("the scheduler made no progress; the cache pool is too small for the queued requests")
            for o in outs:
                results[o.seq_id].extend(o.tokens)
        return [results[i] for i in ids]
