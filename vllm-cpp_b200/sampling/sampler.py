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


class Sampler:
    def __init__(self, device, max_rows: int, vocab: int):
        self.device, self.vocab = device, vocab
        self.cap = max(1, max_rows)
        self.steps_since_check = 0
        self._alloc()

    def _alloc(self):
        n = self.cap
        # one pinned block: temperature, uniform, top_p, penalty (float32) | top_k (int32)
        self.h_float = torch.empty((4, n), dtype=torch.float32, pin_memory=True)
        self.h_int = torch.empty((1, n), dtype=torch.int32, pin_memory=True)
        self.d_float = torch.empty((4, n), dtype=torch.float32, device=self.device)
        self.d_int = torch.empty((1, n), dtype=torch.int32, device=self.device)
        self.d_out = torch.empty(n, dtype=torch.int32, device=self.device)
        self.h_out = torch.empty(n, dtype=torch.int32, pin_memory=True)

    def sample(self, logits: torch.Tensor, rows: List[SamplingRow]) -> List[int]:
        """One token id per row of ``logits`` [len(rows), vocab] (float32, on the device).
        Rows with a repetition penalty are changed in place."""
        m = len(rows)
        if m == 0:
            return []
        if m > self.cap:
            self.cap = m
            self._alloc()
        hf, hi = self.h_float.numpy(), self.h_int.numpy()
        for i, r in enumerate(rows):
            hf[0, i] = r.temperature
            hf[1, i] = r.uniform
            hf[2, i] = r.top_p
            hf[3, i] = r.repetition_penalty
            hi[0, i] = r.top_k
        self.d_float[:, :m].copy_(self.h_float[:, :m], non_blocking=True)
        self.d_int[:, :m].copy_(self.h_int[:, :m], non_blocking=True)
        temperature, uniform = self.d_float[0, :m], self.d_float[1, :m]

        if any(r.repetition_penalty != 1.0 and len(r.generated) for r in rows):
            ids, start = [], [0]
            for r in rows:
                if r.repetition_penalty != 1.0:
                    ids.extend(sorted(set(int(t) for t in r.generated)))
                start.append(len(ids))
            d_ids = torch.tensor(ids if ids else [0], dtype=torch.int32, device=self.device)
            d_start = torch.tensor(start, dtype=torch.int32, device=self.device)
            ops.repetition_penalty(logits, d_ids, d_start, self.d_float[3, :m].contiguous())

        filtered = [i for i, r in enumerate(rows)
                    if r.temperature > 0 and (r.top_p < 1.0 or r.top_k > 0)]
        out = self.d_out[:m]
        ops.sample(logits, temperature.contiguous(), uniform.contiguous(), out)
        if filtered:
            ops.sample_filtered(logits, temperature.contiguous(), uniform.contiguous(),
                                self.d_float[2, :m].contiguous(), self.d_int[0, :m].contiguous(), out)
        self.h_out[:m].copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.steps_since_check += 1
        if self.steps_since_check >= 64:          # a kernel that gave up on a bounded wait says so here
            self.steps_since_check = 0
            ops.check_status()
        return self.h_out[:m].tolist()
