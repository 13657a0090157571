"""Per-request state.

Follows the reference's ``Sequence`` (include/vllm/core/sequence.hpp:11-94):
prompt ids, output ids, status {waiting, running, finished, preempted}, the count
of tokens whose keys and values are in the cache, ``needs_recompute`` after a
preemption, and ``replay_len`` / ``replay_token`` for rebuilding the cache from
the prompt and the outputs so far.  The block table lives in the cache manager
here, not on the sequence.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import List, Optional

from ..sampling.params import SamplingParams


class SequenceStatus(Enum):
    WAITING = 0
    RUNNING = 1
    FINISHED = 2
    PREEMPTED = 3


@dataclass
class Sequence:
    seq_id: int
    prompt_tokens: List[int]
    params: SamplingParams
    arrival: int = 0
    status: SequenceStatus = SequenceStatus.WAITING
    output_tokens: List[int] = field(default_factory=list)
    num_processed_tokens: int = 0
    needs_recompute: bool = False
    finish_reason: Optional[str] = None
    num_preemptions: int = 0

    @property
    def prompt_len(self) -> int:
        return len(self.prompt_tokens)

    @property
    def output_len(self) -> int:
        return len(self.output_tokens)

    @property
    def total_len(self) -> int:
        return len(self.prompt_tokens) + len(self.output_tokens)

    @property
    def replay_len(self) -> int:
        """Tokens to feed again after a preemption before decoding goes on
        (include/vllm/core/sequence.hpp:37): the prompt and all outputs but the last."""
        return self.prompt_len + max(0, self.output_len - 1)

    def replay_token(self, position: int) -> int:
        """Token at ``position`` of prompt + outputs (include/vllm/core/sequence.hpp:38-40)."""
        if position < self.prompt_len:
            return self.prompt_tokens[position]
        return self.output_tokens[position - self.prompt_len]

    @property
    def remaining(self) -> int:
        """Known tokens not yet in the cache.  1 for a request that decodes."""
        return self.total_len - self.num_processed_tokens

    def tokens(self, start: int, count: int) -> List[int]:
        return [self.replay_token(p) for p in range(start, start + count)]

    @property
    def is_finished(self) -> bool:
        return self.status == SequenceStatus.FINISHED
