"""The engine: requests in, tokens out, one step at a time.

API after the reference's ``Engine`` (include/vllm/core/engine.hpp:35-94):
``initialize`` (done by the constructor), ``add_request``, ``step``, ``run``,
``abort_request``, ``pending_requests``.  Requests are token ids here; the
reference tokenizes text inside ``add_request`` (src/core/engine.cpp:83-104), and
text in and out is outside this engine.

One step (src/core/engine.cpp:106-127 is schedule -> prefill -> decode -> sample):
schedule -> one batch through ``ModelRunner.step`` with prompt portions beside
decoded tokens -> sampling on the device for the rows that end a request's known
tokens -> token ids to the host -> append, check stop, free finished requests.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence as Seq

import torch

from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, SamplingRow, splitmix64, uniform_for
from . import factory
from .runner import StepEntry
from .scheduler import Scheduler
from .sequence import Sequence, SequenceStatus


@dataclass
class GenerationOutput:
    """One request's news of one step (include/vllm/core/engine.hpp:22-28, without text)."""
    seq_id: int
    tokens: List[int]
    finished: bool = False
    finish_reason: Optional[str] = None


@dataclass
class StepStats:
    num_tokens: int = 0
    num_decode_tokens: int = 0
    num_prompt_tokens: int = 0
    num_requests: int = 0
    free_pages: int = 0
    preemptions: int = 0


class Engine:
    def __init__(self, config: EngineConfig):
        self.config = config
        self.model, self.cache, self.runner = factory.build(config)
        self.device = self.runner.device
        self.scheduler = Scheduler(self.cache, config.max_num_seqs, config.max_num_batched_tokens,
                                   config.max_tokens_per_step, config.preempted_to_front)
        self.sampler = Sampler(self.device, config.max_num_seqs, self.model.vocab)
        self.sequences: Dict[int, Sequence] = {}
        self._next_id = 0
        self.last_stats = StepStats()
        self.initialized = True

    # ------------------------------------------------------------- requests
    @property
    def max_context(self) -> int:
        """min(max_model_len, max_position_embeddings, cache capacity) (src/core/engine.cpp:90-93)."""
        return min(self.config.max_model_len, self.model.spec.max_position_embeddings,
                   self.cache.num_pages * self.cache.page_size)

    def add_request(self, prompt_token_ids: Seq[int], params: Optional[SamplingParams] = None) -> int:
        """Queue a request; returns its id.  Checks of src/core/engine.cpp:86-101 plus id range."""
        params = (params or SamplingParams()).resolved(self.config, self.model.spec.stop_token_ids)
        ids = [int(t) for t in prompt_token_ids]
        if not ids:
            raise ValueError("prompt must contain at least one token")
        bad = [t for t in ids if not 0 <= t < self.model.vocab]
        if bad:
            raise ValueError(f"prompt holds token id {bad[0]} outside the vocabulary of {self.model.vocab}")
        if len(ids) > self.max_context:
            raise ValueError(f"prompt exceeds the available context length of {self.max_context} tokens")
        if params.max_tokens > self.max_context - len(ids):
            raise ValueError("prompt tokens plus max_tokens exceeds the available context length of "
                             f"{self.max_context} tokens")
        seq = Sequence(self._next_id, ids, params, arrival=self._next_id)
        if params.seed is None:
            params.seed = splitmix64((self.config.seed << 20) ^ seq.seq_id)
        self.scheduler.add_request(seq)
        self.sequences[seq.seq_id] = seq
        self._next_id += 1
        return seq.seq_id

    def abort_request(self, seq_id: int) -> None:
        self.scheduler.abort_request(seq_id)
        self.sequences.pop(seq_id, None)

    def pending_requests(self) -> int:
        return len(self.scheduler.waiting) + len(self.scheduler.running)

    def has_pending_work(self) -> bool:
        return self.scheduler.has_pending_work()

    # ----------------------------------------------------------------- step
    def step(self) -> List[GenerationOutput]:
        items = self.scheduler.schedule()
        if not items:
            return []
        entries, sampled = [], []
        stats = StepStats(num_requests=len(items))
        for it in items:
            toks = it.seq.tokens(it.start, it.count)
            entries.append(StepEntry(it.seq.seq_id, toks, [it.count - 1] if it.samples else []))
            stats.num_tokens += it.count
            if it.count == 1:
                stats.num_decode_tokens += 1
            else:
                stats.num_prompt_tokens += it.count
            if it.samples:
                sampled.append(it.seq)
        with torch.no_grad():
            logits = self.runner.step(entries)
            rows = [SamplingRow(s.params.temperature, s.params.top_p, s.params.top_k,
                                s.params.repetition_penalty, s.output_tokens,
                                uniform_for(s.params.seed, s.output_len)) for s in sampled]
            tokens = self.sampler.sample(logits, rows)
        for it in items:
            it.seq.num_processed_tokens += it.count
        outputs = []
        for seq, tok in zip(sampled, tokens):
            seq.output_tokens.append(tok)
            reason = None
            if not seq.params.ignore_eos and tok in seq.params.stop_token_ids:
                reason = "stop"
            elif seq.output_len >= seq.params.max_tokens:
                reason = "length"
            if reason:
                self.scheduler.finish_sequence(seq, reason)
                self.sequences.pop(seq.seq_id, None)
            outputs.append(GenerationOutput(seq.seq_id, [tok], reason is not None, reason))
        stats.free_pages = self.cache.num_free_pages()
        stats.preemptions = self.scheduler.num_preemptions
        self.last_stats = stats
        return outputs

    def run(self, callback: Optional[Callable[[GenerationOutput], None]] = None) -> None:
        """Step until nothing is pending (src/core/engine.cpp:129-136)."""
        while self.scheduler.has_pending_work():
            for out in self.step():
                if callback:
                    callback(out)
