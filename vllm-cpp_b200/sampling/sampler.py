"""Sampling on the device for the rows of a step's logits.

Order of operations as in the reference's ``Sampler::sample``
(src/sampler/sampler.cpp:23-79): repetition penalty over the unique ids generated
so far, temperature, greedy when temperature <= 0, else softmax, top-k, top-p and
an inverse-CDF draw.  The kernels are in csrc/sampling.cu; only the chosen token
ids are copied to the host.

The uniform number of a draw comes from a counter-based generator keyed by the
request's seed and the index of the token being drawn, so a request's tokens do
not depend on what else is in the batch or on how its prompt was cut.  (The
reference draws from a thread-local mt19937 seeded by random_device, sampler.cpp:68.)
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from ..csrc import ops

_MASK64 = (1 << 64) - 1


def splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK64
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    return z ^ (z >> 31)


def uniform_for(seed: int, index: int) -> float:
    """The uniform number in [0, 1) of draw ``index`` of a request with ``seed``: 24 random bits."""
    h = splitmix64(splitmix64(seed & _MASK64) ^ ((index + 1) * 0xD1342543DE82EF95 & _MASK64))
    return (h >> 40) / float(1 << 24)


class SamplingRow:
    """What the sampler needs to know about one logits row."""
    __slots__ = ("temperature", "top_p", "top_k", "repetition_penalty", "generated", "uniform")

    def __init__(self, temperature: float, top_p: float, top_k: int, repetition_penalty: float,
                 generated: Sequence[int], uniform: float):
        self.temperature, self.top_p, self.top_k = temperature, top_p, top_k
        self.repetition_penalty, self.generated, self.uniform = repetition_penalty, generated, uniform


class SampleHandle:
    """A sampling whose kernels and copy have been enqueued; ``Sampler.wait`` gives its token ids."""
    __slots__ = ("slot", "m", "event")

    def __init__(self, slot: int, m: int, event):
        self.slot, self.m, self.event = slot, m, event


class Sampler:
    """``sample`` = ``launch`` + ``wait``.  Two launches may be in flight (the engine launches the
    next step before it reads this step's tokens), so the pinned host buffers exist twice."""
    SLOTS = 2

    def __init__(self, device, max_rows: int, vocab: int):
        self.device, self.vocab = device, vocab
        self.cap = max(1, max_rows)
        self.steps_since_check = 0
        self._slot = 0
        self._alloc()

    def _alloc(self):
        n = self.cap
        # one pinned block per slot: temperature, uniform, top_p, penalty (float32) | top_k (int32)
        self.h_float = [torch.empty((4, n), dtype=torch.float32, pin_memory=True) for _ in range(self.SLOTS)]
        self.h_int = [torch.empty((1, n), dtype=torch.int32, pin_memory=True) for _ in range(self.SLOTS)]
        self.h_out = [torch.empty(n, dtype=torch.int32, pin_memory=True) for _ in range(self.SLOTS)]
        self.d_float = [torch.empty((4, n), dtype=torch.float32, device=self.device) for _ in range(self.SLOTS)]
        self.d_int = [torch.empty((1, n), dtype=torch.int32, device=self.device) for _ in range(self.SLOTS)]
        self.d_out = [torch.empty(n, dtype=torch.int32, device=self.device) for _ in range(self.SLOTS)]
        self.events = [torch.cuda.Event() for _ in range(self.SLOTS)]

    def device_ids(self, handle: SampleHandle) -> torch.Tensor:
        """The sampled ids of ``handle`` on the device (valid in stream order after its launch)."""
        return self.d_out[handle.slot][: handle.m]

    def launch(self, logits: torch.Tensor, rows: List[SamplingRow]) -> SampleHandle:
        """Enqueue the sampling of one token id per row of ``logits`` [len(rows), vocab] (float32, on
        the device) and the copy of the ids to the host.  Rows with a repetition penalty are changed
        in place."""
        m = len(rows)
        if m > self.cap:
            torch.cuda.current_stream().synchronize()      # nothing may be in flight in the old buffers
            self.cap = m
            self._alloc()
        slot = self._slot
        self._slot = (slot + 1) % self.SLOTS
        if m == 0:
            return SampleHandle(slot, 0, None)
        hf, hi = self.h_float[slot].numpy(), self.h_int[slot].numpy()
        for i, r in enumerate(rows):
            hf[0, i] = r.temperature
            hf[1, i] = r.uniform
            hf[2, i] = r.top_p
            hf[3, i] = r.repetition_penalty
            hi[0, i] = r.top_k
        filtered = [i for i, r in enumerate(rows)
                    if r.temperature > 0 and (r.top_p < 1.0 or r.top_k > 0)]
        d_float, d_int = self.d_float[slot], self.d_int[slot]
        d_float[:, :m].copy_(self.h_float[slot][:, :m], non_blocking=True)
        if filtered:                                       # only the filtered draw reads top_k
            d_int[:, :m].copy_(self.h_int[slot][:, :m], non_blocking=True)
        temperature, uniform = d_float[0, :m], d_float[1, :m]

        if any(r.repetition_penalty != 1.0 and len(r.generated) for r in rows):
            ids, start = [], [0]
            for r in rows:
                if r.repetition_penalty != 1.0:
                    ids.extend(sorted(set(int(t) for t in r.generated)))
                start.append(len(ids))
            d_ids = torch.tensor(ids if ids else [0], dtype=torch.int32, device=self.device)
            d_start = torch.tensor(start, dtype=torch.int32, device=self.device)
            ops.repetition_penalty(logits, d_ids, d_start, d_float[3, :m].contiguous())

        out = self.d_out[slot][:m]
        ops.sample(logits, temperature.contiguous(), uniform.contiguous(), out)
        if filtered:
            ops.sample_filtered(logits, temperature.contiguous(), uniform.contiguous(),
                                d_float[2, :m].contiguous(), d_int[0, :m].contiguous(), out)
        self.h_out[slot][:m].copy_(out, non_blocking=True)
        self.events[slot].record()
        return SampleHandle(slot, m, self.events[slot])

    def wait(self, handle: SampleHandle) -> List[int]:
        """The token ids of a launched sampling (blocks until its copy has arrived)."""
        if handle.m == 0:
            return []
        handle.event.synchronize()
        self.steps_since_check += 1
        if self.steps_since_check >= 64:          # a kernel that gave up on a bounded wait says so here
            self.steps_since_check = 0
            ops.check_status()
        return self.h_out[handle.slot][: handle.m].tolist()

    def sample(self, logits: torch.Tensor, rows: List[SamplingRow]) -> List[int]:
        """One token id per row of ``logits``: ``launch`` and ``wait`` in one."""
        return self.wait(self.launch(logits, rows))
