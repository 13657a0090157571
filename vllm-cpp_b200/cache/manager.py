"""The cache manager: paged keys and values with a block table per request, in
groups of layers with the same needs, and slots for per-request state of fixed size.

The reference keeps one pool of blocks for all layers, a ``vector<int32>`` block
table on each Sequence (include/vllm/core/sequence.hpp:54-55) and grows it with
``ensure_sequence_capacity`` with rollback (src/core/block_manager.cpp:82-97);
blocks go back on finish, abort and preemption (src/core/scheduler.cpp:111-121,
168-188).  It has one kind of layer and no per-request state.

Here cache layers whose mixers declare the same PagedKVSpec (kv heads, head size,
window) form a group with pages and tables of its own.  A request holds one table
per group.  A group with a window gives pages back as soon as the window has
passed them: a query at position p reads keys j with p - window < j <= p, so once
a request holds ``n`` tokens no later query reads a key at or below n - window.
Layers that declare a StateSpec get one slot per live request in a tensor of
their own; the slot is zeroed when the request is admitted.  A request always
gets a slot id, even if no layer has state.

All bookkeeping is host-side and runs without a GPU (``device=None``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch

from ..parts.base import PagedKVSpec, PagedKVView, StateSpec, StateView
from .block_pool import BlockPool, PageError

RELEASED = -1     # table entry of a page that a window has passed


class OutOfPages(RuntimeError):
    """A request's next tokens do not fit the free pages of some group."""


@dataclass
class PagedGroup:
    spec: PagedKVSpec
    layers: List[int]                      # cache layer ids, in order
    pool: BlockPool
    pages: Optional[torch.Tensor] = None   # [len(layers), num_pages, 2, kv_heads, page_size * head_dim]: see csrc/common.cuh (kv_pos)


@dataclass
class StateGroup:
    spec: StateSpec
    layers: List[int]
    slots: Optional[torch.Tensor] = None   # [len(layers), num_slots, *shape]


@dataclass
class RequestCache:
    tables: List[List[int]]                # one per paged group
    num_tokens: int = 0
    slot: int = -1
    released: List[int] = field(default_factory=list)   # per group: blocks [0, released) are given back


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


class CacheManager:
    def __init__(self, cache_specs: List[object], page_size: int, num_pages: int, max_num_seqs: int,
                 dtype: torch.dtype = torch.float32, device=None):
        if page_size <= 0:
            raise ValueError("KV block size must be greater than zero")
        self.page_size, self.num_pages, self.max_num_seqs = page_size, num_pages, max_num_seqs
        self.dtype, self.device = dtype, device
        self.paged: List[PagedGroup] = []
        self.state: List[StateGroup] = []
        self._where: List[Optional[tuple]] = []          # cache layer -> ("paged"|"state", group, index in group)
        for layer, spec in enumerate(cache_specs):
            if spec is None:
                self._where.append(None)
            elif isinstance(spec, PagedKVSpec):
                g = next((i for i, pg in enumerate(self.paged) if pg.spec == spec), None)
                if g is None:
                    self.paged.append(PagedGroup(spec, [], BlockPool(num_pages)))
                    g = len(self.paged) - 1
                self._where.append(("paged", g, len(self.paged[g].layers)))
                self.paged[g].layers.append(layer)
            elif isinstance(spec, StateSpec):
                g = next((i for i, sg in enumerate(self.state) if sg.spec == spec), None)
                if g is None:
                    self.state.append(StateGroup(spec, []))
                    g = len(self.state) - 1
                self._where.append(("state", g, len(self.state[g].layers)))
                self.state[g].layers.append(layer)
            else:
                raise TypeError(f"cache layer {layer}: unknown cache need {spec!r}")
        self._free_slots: List[int] = list(range(max_num_seqs - 1, -1, -1))
        self.requests: Dict[object, RequestCache] = {}
        # every group's block tables as rows of one array (see table_rows); widened on demand
        self._table_rows: List[np.ndarray] = [np.full((max_num_seqs, 0), RELEASED, dtype=np.int32) for _ in self.paged]
        if device is not None:
            self._allocate_device()

    # ---------------------------------------------------------------- device
    @staticmethod
    def bytes_per_page(cache_specs: List[object], page_size: int, dtype: torch.dtype) -> int:
        """Device bytes that one page id costs over all paged cache layers."""
        el = torch.empty((), dtype=dtype).element_size()
        return sum(2 * s.num_kv_heads * page_size * s.head_dim * el
                   for s in cache_specs if isinstance(s, PagedKVSpec))

    def _allocate_device(self) -> None:
        for g in self.paged:
            s = g.spec
            g.pages = torch.zeros((len(g.layers), self.num_pages, 2, s.num_kv_heads, self.page_size * s.head_dim),
                                  dtype=self.dtype, device=self.device)
        for g in self.state:
            g.slots = torch.zeros((len(g.layers), self.max_num_seqs) + tuple(g.spec.shape),
                                  dtype=g.spec.dtype, device=self.device)

    def views(self) -> List[object]:
        """What each cache layer's mixer is handed."""
        out = []
        for w in self._where:
            if w is None:
                out.append(None)
            elif w[0] == "paged":
                g = self.paged[w[1]]
                out.append(PagedKVView(g.pages[w[2]] if g.pages is not None else None, w[1], self.page_size))
            else:
                g = self.state[w[1]]
                out.append(StateView(g.slots[w[2]] if g.slots is not None else None))
        return out

    # ------------------------------------------------------------- requests
    def has_free_slot(self) -> bool:
        return bool(self._free_slots)

    def add_request(self, req_id) -> RequestCache:
        if req_id in self.requests:
            raise KeyError(f"request {req_id!r} is already live")
        if not self._free_slots:
            raise OutOfPages(f"all {self.max_num_seqs} request slots are taken")
        slot = self._free_slots.pop()
        rc = RequestCache(tables=[[] for _ in self.paged], slot=slot, released=[0] * len(self.paged))
        self.requests[req_id] = rc
        for t in self._table_rows:
            t[slot, :] = RELEASED
        for g in self.state:
            if g.slots is not None:
                g.slots[:, slot].zero_()
        return rc

    def pages_needed(self, req_id, n_new: int) -> List[int]:
        """Pages each group must still hand out before ``n_new`` more tokens fit."""
        rc = self.requests[req_id]
        want = cdiv(rc.num_tokens + n_new, self.page_size)
        return [max(0, want - len(t)) for t in rc.tables]

    def can_append(self, req_id, n_new: int) -> bool:
        return all(g.pool.can_allocate(n) for g, n in zip(self.paged, self.pages_needed(req_id, n_new)))

    def max_appendable(self, req_id=None) -> int:
        """Most tokens that the request (or, with None, a new request) could take now."""
        if not self.paged:
            return 1 << 30
        if req_id is None:
            return self.num_free_pages() * self.page_size
        rc = self.requests[req_id]
        return min((len(t) + g.pool.num_free) * self.page_size for g, t in zip(self.paged, rc.tables)) \
            - rc.num_tokens

    def reserve(self, req_id, n_new: int) -> None:
        """Give the request pages for its next ``n_new`` tokens in every group, or none at all."""
        rc = self.requests[req_id]
        need = self.pages_needed(req_id, n_new)
        for g, n in zip(self.paged, need):
            if not g.pool.can_allocate(n):
                raise OutOfPages(f"request {req_id!r} needs {n} more pages for {n_new} tokens; "
                                 f"{g.pool.num_free} of {self.num_pages} are free")
        for gi, (g, table, n) in enumerate(zip(self.paged, rc.tables, need)):
            for _ in range(n):
                page = g.pool.acquire()
                if len(table) < self._table_rows[gi].shape[1]:
                    self._table_rows[gi][rc.slot, len(table)] = page
                table.append(page)

    def commit(self, req_id, n_new: int) -> None:
        """The request now holds ``n_new`` more tokens; give back what windows have passed."""
        rc = self.requests[req_id]
        rc.num_tokens += n_new
        if rc.tables and rc.num_tokens > min(len(t) for t in rc.tables) * self.page_size:
            raise PageError(f"request {req_id!r} holds {rc.num_tokens} tokens but pages for fewer")
        for gi, g in enumerate(self.paged):
            w = g.spec.window
            if w <= 0:
                continue
            # keys at positions <= num_tokens - w are never read again
            dead_blocks = max(0, (rc.num_tokens - w + 1) // self.page_size)
            table = rc.tables[gi]
            for b in range(rc.released[gi], min(dead_blocks, len(table))):
                g.pool.release(table[b])
                table[b] = RELEASED
                if b < self._table_rows[gi].shape[1]:
                    self._table_rows[gi][rc.slot, b] = RELEASED
            rc.released[gi] = max(rc.released[gi], min(dead_blocks, len(table)))

    def free_request(self, req_id) -> None:
        rc = self.requests.pop(req_id)
        for g, table in zip(self.paged, rc.tables):
            for b in reversed(table):
                if b != RELEASED:
                    g.pool.release(b)
        self._free_slots.append(rc.slot)

    # ---------------------------------------------------------------- queries
    def num_tokens(self, req_id) -> int:
        return self.requests[req_id].num_tokens

    def table(self, req_id, group: int) -> List[int]:
        return self.requests[req_id].tables[group]

    def table_rows(self, group: int, width: int) -> np.ndarray:
        """The block tables of the group as one int32 array [request slot, width], kept up to date
        with every page handed out or given back (RELEASED where a request holds no page): the
        step function copies rows of it instead of building tables from lists."""
        rows = self._table_rows[group]
        if rows.shape[1] < width:
            wider = np.full((self.max_num_seqs, width), RELEASED, dtype=np.int32)
            for rc in self.requests.values():
                t = rc.tables[group][:width]
                wider[rc.slot, : len(t)] = t
            self._table_rows[group] = rows = wider
        return rows

    def slot(self, req_id) -> int:
        return self.requests[req_id].slot

    def num_free_pages(self) -> int:
        """Free pages of the scarcest group."""
        return min((g.pool.num_free for g in self.paged), default=self.num_pages)
