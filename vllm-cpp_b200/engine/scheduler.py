"""Continuous batching with token-budgeted portions of prompts.

Shape of the reference's Scheduler (src/core/scheduler.cpp:14-188): a FCFS waiting
queue, a running list, ``add_request`` / ``schedule`` / ``finish_sequence`` /
``abort_request``, and preemption by recompute: the newest running request loses
all its pages, keeps its outputs, and later feeds prompt and outputs again
(:168-188).  What differs, and why:

* The reference's budget counts sequences, and a new request's whole prompt runs
  inside one step (src/core/scheduler.cpp:94-98, src/core/engine.cpp:157-164).
  Here the budgets count tokens: a step holds at most ``max_num_batched_tokens``
  tokens, of which at most ``max_tokens_per_step`` belong to portions of more than
  one token; a prompt is cut into portions of whatever size the budgets and the
  free pages allow.
* Pages are taken per portion, not for the whole prompt at admission (:147-166).
* A waiting request never preempts a running one (the reference does, :57).  Only
  a decoding request that needs its next page preempts, newest victim first,
  never itself (:73-83) and, unlike the reference, never a request admitted before
  it: the newest request sits a step out instead of evicting an older one.  If
  nothing at all can run while requests are running (all of them mid-prompt and
  the pages gone), the newest is preempted so that the others can finish.
* A request that is re-admitted after preemption feeds prompt + outputs in
  portions like a prompt; the portion that reaches its last known token is
  sampled from, so no separate decode step is needed after the replay
  (the reference replays ``replay_len`` tokens, then decodes, src/core/engine.cpp:165-166).
* Finished requests leave the running list at once (the reference never erases them).

When pages run out, in short: decoding requests win over requests still reading
their prompt, older requests win over newer ones, and a preempted request goes to
the back of the waiting queue (the reference's choice, :183) or to its front
(``preempted_to_front``).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Deque, List, Optional

from .sequence import Sequence, SequenceStatus


@dataclass
class ScheduledItem:
    seq: Sequence
    start: int            # position of the first token of this portion
    count: int            # tokens in this portion
    samples: bool         # the portion reaches the last known token: a token is sampled


class Scheduler:
    def __init__(self, cache, max_num_seqs: int, max_num_batched_tokens: int, max_tokens_per_step: int,
                 preempted_to_front: bool = False):
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_tokens_per_step = max_tokens_per_step
        self.preempted_to_front = preempted_to_front
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self.num_preemptions = 0

    # ------------------------------------------------------------- requests
    def add_request(self, seq: Sequence) -> None:
        """Queue a request.  Refused if prompt + max_tokens can never fit the pool
        (src/core/scheduler.cpp:20-26), which guarantees that a request alone can finish."""
        if seq.prompt_len == 0:
            raise ValueError("prompt must contain at least one token")
        planned = seq.prompt_len + seq.params.max_tokens
        page = self.cache.page_size
        if -(-planned // page) > self.cache.num_pages:
            raise ValueError("request exceeds total KV cache block capacity")
        self.waiting.append(seq)

    def has_pending_work(self) -> bool:
        return bool(self.waiting) or bool(self.running)

    def finish_sequence(self, seq: Sequence, reason: str) -> None:
        seq.status = SequenceStatus.FINISHED
        seq.finish_reason = reason
        if seq in self.running:
            self.running.remove(seq)
            self.cache.free_request(seq.seq_id)
        elif seq in self.waiting:
            self.waiting.remove(seq)

    def abort_request(self, seq_id: int) -> bool:
        for seq in list(self.running) + list(self.waiting):
            if seq.seq_id == seq_id:
                self.finish_sequence(seq, "abort")
                return True
        return False

    # ------------------------------------------------------------- schedule
    def schedule(self) -> List[ScheduledItem]:
        """The next step's batch.  Pages for every item are reserved before it returns."""
        while True:
            items = self._schedule_once()
            if items or not self.running:
                return items
            # Requests are running but none got a token: the pages are gone and nobody
            # decodes.  Take the newest one's pages so that the others can go on.
            victim = self._newest_running(newer_than=None)
            if victim is None or len(self.running) == 1 and not self._could_ever_run(victim):
                return items
            self._preempt(victim, items)

    def _could_ever_run(self, seq: Sequence) -> bool:
        return self.cache.max_appendable(seq.seq_id) > 0

    def _schedule_once(self) -> List[ScheduledItem]:
        items: List[ScheduledItem] = []
        budget = self.max_num_batched_tokens
        portion_budget = self.max_tokens_per_step

        # 1. requests that decode: one token each, oldest first; may preempt the newest
        i = 0
        while i < len(self.running):
            seq = self.running[i]
            if seq.remaining == 1 and budget > 0:
                while not self.cache.can_append(seq.seq_id, 1):
                    victim = self._newest_running(newer_than=seq)
                    if victim is None:
                        break          # nobody newer to take pages from: sit this step out
                    budget += self._preempt(victim, items)
                if self.cache.can_append(seq.seq_id, 1):
                    self.cache.reserve(seq.seq_id, 1)
                    items.append(ScheduledItem(seq, seq.num_processed_tokens, 1, True))
                    budget -= 1
            i += 1

        # 2. running requests still reading their prompt (or replaying), in arrival order
        for seq in self.running:
            if seq.remaining > 1 and budget > 0 and portion_budget > 0:
                n = min(seq.remaining, budget, portion_budget, self.cache.max_appendable(seq.seq_id))
                if n <= 0:
                    continue
                self.cache.reserve(seq.seq_id, n)
                items.append(ScheduledItem(seq, seq.num_processed_tokens, n, n == seq.remaining))
                budget -= n
                if n > 1:
                    portion_budget -= n

        # 3. admissions, strictly in queue order
        while (self.waiting and len(self.running) < self.max_num_seqs and budget > 0
               and self.cache.has_free_slot()):
            seq = self.waiting[0]
            n = min(seq.remaining, budget, portion_budget if seq.remaining > 1 else 1)
            if n <= 0 or self.cache.max_appendable(None) < n:
                break
            self.waiting.popleft()
            self.cache.add_request(seq.seq_id)
            self.cache.reserve(seq.seq_id, n)
            seq.status = SequenceStatus.RUNNING
            seq.needs_recompute = False
            self.running.append(seq)
            items.append(ScheduledItem(seq, 0, n, n == seq.remaining))
            budget -= n
            if n > 1:
                portion_budget -= n
        return items

    # ----------------------------------------------------------- preemption
    def _newest_running(self, newer_than: Optional[Sequence]) -> Optional[Sequence]:
        """The most recently admitted running request, if it was admitted after ``newer_than``."""
        if not self.running or self.running[-1] is newer_than:
            return None
        return self.running[-1]

    def _preempt(self, victim: Sequence, items: List[ScheduledItem]) -> int:
        """Recompute-style preemption (src/core/scheduler.cpp:168-188).  Returns the
        tokens of the step's budget that the victim had been given."""
        freed = 0
        for it in list(items):
            if it.seq is victim:
                items.remove(it)
                freed += it.count
        self.running.remove(victim)
        self.cache.free_request(victim.seq_id)
        victim.num_processed_tokens = 0
        victim.needs_recompute = True
        victim.status = SequenceStatus.PREEMPTED
        victim.num_preemptions += 1
        self.num_preemptions += 1
        if self.preempted_to_front:
            self.waiting.appendleft(victim)
        else:
            self.waiting.append(victim)
        return freed
