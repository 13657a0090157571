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

While every running request decodes, the step after is launched before this step's tokens
are read (``overlap_decode_steps``): its metadata depends on lengths only, and the token
ids reach it on the device.  ``step`` still returns one step's news per call, in order; a
request that turns out to have ended leaves one unused row in the step launched ahead.
"""
from __future__ import annotations

import time
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
    # with EngineConfig.time_phases: milliseconds of this step's phases.  Host time: "schedule", "pack"
    # (metadata into the pinned buffer and its copy enqueued), "launch" (the model's kernels enqueued),
    # "sample" (sampling and the read-back enqueued), "wait" (blocked until the token ids arrived).
    # Device time, between CUDA events: "device_forward", "device_sample".
    phase_ms: Dict[str, float] = field(default_factory=dict)


@dataclass
class _InFlight:
    """A step that is on the device: what was scheduled, who gets a token, where in their outputs."""
    items: list
    sampled: List[Sequence]
    slots: List[int]
    handle: object
    stats: StepStats
    events: Optional[tuple] = None        # (before the forward, after it, after the sampling) when phases are timed


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
        self._ahead: Optional[_InFlight] = None       # a step launched before the one before it was read
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
    PLACEHOLDER = -1          # stands in a request's outputs for a token that is still on the device

    def _launch(self, items, token_source=None) -> "_InFlight":
        """Send one scheduled batch to the device: model, sampling, copy of the ids; nothing is waited for."""
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
        timers = {} if self.config.time_phases else None
        events = None
        with torch.no_grad():
            logits = self.runner.step(entries, device_tokens=token_source, timers=timers)
            if timers is not None:
                after_forward = torch.cuda.Event(enable_timing=True)
                after_forward.record()
                t0 = time.perf_counter()
            rows = [SamplingRow(s.params.temperature, s.params.top_p, s.params.top_k,
                                s.params.repetition_penalty, s.output_tokens,
                                uniform_for(s.params.seed, s.output_len)) for s in sampled]
            handle = self.sampler.launch(logits, rows)
            if timers is not None:
                after_sample = torch.cuda.Event(enable_timing=True)
                after_sample.record()
                events = (timers["forward_start"], after_forward, after_sample)
                stats.phase_ms.update(pack=timers["pack"] * 1e3, launch=timers["launch"] * 1e3,
                                      sample=(time.perf_counter() - t0) * 1e3)
        for it in items:
            it.seq.num_processed_tokens += it.count
        # the token each sampled request will get: known to the host at _collect
        slots = []
        for seq in sampled:
            slots.append(seq.output_len)
            seq.output_tokens.append(self.PLACEHOLDER)
        return _InFlight(items, sampled, slots, handle, stats, events)

    def _may_run_ahead(self, flight: "_InFlight") -> bool:
        """True if the step after ``flight`` is known without its tokens: every running request took
        part with one token and will go on (no length limit reached, no waiting request to admit,
        no repetition penalty, which needs the ids on the host)."""
        if not self.config.overlap_decode_steps or self.scheduler.waiting:
            return False
        if len(flight.items) != len(self.scheduler.running) or len(flight.sampled) != len(flight.items):
            return False
        for it in flight.items:
            seq = it.seq
            if it.count != 1 or seq.output_len >= seq.params.max_tokens or seq.params.repetition_penalty != 1.0:
                return False
        return True

    def _collect(self, flight: "_InFlight") -> List[GenerationOutput]:
        """Wait for the step's token ids, put them where the placeholders stand, check the stops."""
        t0 = time.perf_counter()
        tokens = self.sampler.wait(flight.handle)
        if flight.events is not None:
            before, after_forward, after_sample = flight.events
            after_sample.synchronize()
            flight.stats.phase_ms.update(wait=(time.perf_counter() - t0) * 1e3,
                                         device_forward=before.elapsed_time(after_forward),
                                         device_sample=after_forward.elapsed_time(after_sample))
        outputs = []
        for seq, slot, tok in zip(flight.sampled, flight.slots, tokens):
            if seq.is_finished:
                continue                  # ended (or was aborted) while this step was already on its way
            seq.output_tokens[slot] = tok
            reason = None
            if not seq.params.ignore_eos and tok in seq.params.stop_token_ids:
                reason = "stop"
            elif slot + 1 >= seq.params.max_tokens:
                reason = "length"
            if reason:
                del seq.output_tokens[slot + 1:]          # a placeholder of a step launched ahead
                self.scheduler.finish_sequence(seq, reason)
                self.sequences.pop(seq.seq_id, None)
            outputs.append(GenerationOutput(seq.seq_id, [tok], reason is not None, reason))
        flight.stats.free_pages = self.cache.num_free_pages()
        flight.stats.preemptions = self.scheduler.num_preemptions
        self.last_stats = flight.stats
        return outputs

    def step(self) -> List[GenerationOutput]:
        flight, self._ahead = self._ahead, None
        if flight is None:
            t0 = time.perf_counter()
            items = self.scheduler.schedule()
            if not items:
                self.last_stats = StepStats()
                return []
            scheduled_ms = (time.perf_counter() - t0) * 1e3
            flight = self._launch(items)
            if self.config.time_phases:
                flight.stats.phase_ms["schedule"] = scheduled_ms
        if self._may_run_ahead(flight):
            t0 = time.perf_counter()
            items = self.scheduler.schedule()
            scheduled_ms = (time.perf_counter() - t0) * 1e3
            # only a plain continuation is sent ahead: the same requests, in the same order, one token each
            if len(items) == len(flight.sampled) and all(
                    it.seq is s and it.count == 1 and it.samples for it, s in zip(items, flight.sampled)):
                self._ahead = self._launch(items, token_source=self.sampler.device_ids(flight.handle))
                if self.config.time_phases:
                    self._ahead.stats.phase_ms["schedule"] = scheduled_ms
            elif items:
                # Not a plain continuation (pages ran short: somebody sits out or was preempted).  The
                # batch is scheduled, so it runs, but only once this step's tokens are known.
                outputs = self._collect(flight)
                items = [it for it in items if not it.seq.is_finished]
                if items:
                    self._ahead = self._launch(items)
                return outputs
        return self._collect(flight)

    def run(self, callback: Optional[Callable[[GenerationOutput], None]] = None) -> None:
        """Step until nothing is pending (src/core/engine.cpp:129-136)."""
        while self.scheduler.has_pending_work():
            for out in self.step():
                if callback:
                    callback(out)
