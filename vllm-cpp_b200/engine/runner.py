"""The step function: one batch of (request, its next tokens) through the model.

``ModelRunner.step`` takes, for each request in the batch, the tokens it brings
now (a portion of a prompt of any length, or one decoded token) and the places
among them whose logits are wanted.  It runs exactly those tokens, as one batch,
against what earlier steps left in the cache, and returns float32 logits for the
wanted places only.  The scheduler-driven engine and the replay tool both call
it; there is no other forward path.

The reference's counterpart is ``ModelBase::forward(logits, ids, batch, &ctx,
block_table)`` (include/vllm/model/model_registry.hpp:15-16), which in practice
takes one token of one sequence (src/core/engine.cpp:157-164,176-187) and uploads
the context length and block table once per layer (src/layers/attention.cpp:105-110).
Here all of a step's metadata is packed into one pinned buffer and copied to the
device once.

Device memory is static: the metadata buffer, the workspace and the logits buffer
are allocated once, so a pure-decode step of a given batch size touches the same
addresses every time and can be replayed as a CUDA graph.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import time

import numpy as np
import torch

from ..cache.manager import CacheManager, cdiv
from ..parts.base import StepContext, Workspace
from .memory_plan import MAX_CAPTURED_STEPS


@dataclass
class StepEntry:
    req_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()          # places among ``tokens`` whose logits are returned


@dataclass
class HostStep:
    """Host-side facts of a step, handed to the parts' work-list builders."""
    q_lens: List[int]
    ctx_lens: List[int]               # tokens in the cache before the step
    page_size: int
    # launch shapes (grid sizes and the like) that a builder derives from the step: a captured step is
    # replayed only for steps with the same shapes
    shapes: Dict[str, int] = field(default_factory=dict)


class StepError(ValueError):
    pass


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class ModelRunner:
    def __init__(self, model, cache: CacheManager, max_num_batched_tokens: int, max_num_seqs: int,
                 max_model_len: int, device, use_cuda_graphs: bool = False, workspace_bytes: int = 0):
        self.model, self.cache, self.device = model, cache, device
        self.max_tokens, self.max_seqs, self.max_model_len = max_num_batched_tokens, max_num_seqs, max_model_len
        self.max_blocks = cdiv(max_model_len, cache.page_size)
        self.n_groups = len(cache.paged)
        self.views = cache.views()
        self.ws = Workspace(device, workspace_bytes)      # at its planned size it never grows
        self.memory_plan = None
        self.logits = torch.empty((max(1, max_num_seqs), model.vocab), dtype=torch.float32, device=device)
        # work lists that parts ask for: name -> builder(HostStep) -> int32 numpy array
        self.array_builders: Dict[str, Callable[[HostStep], np.ndarray]] = {}
        for owner in [p for blk in model.blocks for p in (blk, *blk.parts.values())] + [model.final_norm]:
            builders = getattr(owner, "step_arrays", None)
            if builders:
                self.array_builders.update(builders())
            reserve = getattr(owner, "reserve", None)
            if reserve and torch.device(device).type == "cuda":
                reserve(max_num_batched_tokens, max_num_seqs, device)
        cap = self._meta_ints(self.max_tokens, self.max_seqs, self.max_tokens) + 64 * 1024
        self.meta_host = torch.empty(cap, dtype=torch.int32, pin_memory=True)
        self.meta_dev = torch.empty(cap, dtype=torch.int32, device=device)
        self._copy_done = torch.cuda.Event()
        self._copy_pending = False
        self.use_cuda_graphs = use_cuda_graphs
        self.graphs: Dict[tuple, object] = {}
        self._graph_seen: Dict[tuple, int] = {}
        self._graph_sig = None
        self.last_meta_bytes = 0

    def _meta_ints(self, n: int, r: int, m: int) -> int:
        return (3 * _align(n) + _align(r + 1) + 2 * _align(r) + _align(m)
                + self.n_groups * _align(r * self.max_blocks))

    # ------------------------------------------------------------------ step
    def step(self, entries: List[StepEntry], device_tokens: Optional[torch.Tensor] = None,
             timers: Optional[dict] = None) -> torch.Tensor:
        """Run one batch; returns float32 logits [number of wanted places, vocab] on the device,
        in the order of the entries and of each entry's ``want``.  The tensor is a
        view of the runner's logits buffer and is overwritten by the next step.
        ``device_tokens``: int32 ids on the device, one per entry of a step in which every entry
        brings one token; they replace the entries' token ids (which are then not looked at) in
        stream order, for a step launched before the ids it continues from have reached the host.
        ``timers``: a dict that receives the host seconds of packing the metadata ("pack") and of
        enqueuing the model's kernels ("launch"), and a CUDA event recorded before the first of them
        ("forward_start")."""
        t0 = time.perf_counter() if timers is not None else 0.0
        step = self._prepare(entries, ids_on_device=device_tokens is not None)
        if timers is not None:
            t1 = time.perf_counter()
            timers["pack"] = t1 - t0
            timers["forward_start"] = torch.cuda.Event(enable_timing=True)
            timers["forward_start"].record()
        if device_tokens is not None:
            if not step.decode_only or device_tokens.numel() != step.n_tokens:
                raise StepError("device_tokens needs one token per entry")
            step.token_ids.copy_(device_tokens, non_blocking=True)
        if self.use_cuda_graphs and step.decode_only and step.n_logit_rows == step.n_reqs:
            out = self._run_decode_graph(step)
        else:
            self.ws.reset()
            out = self.model.forward(step, self.views, self.ws, self.logits)
        for e in entries:
            self.cache.commit(e.req_id, len(e.tokens))
        if timers is not None:
            timers["launch"] = time.perf_counter() - t1
        return out

    # ---------------------------------------------------------- CUDA graphs
    def _buffers_signature(self):
        from ..csrc import ops
        return (self.meta_dev.data_ptr(), self.ws.buf.data_ptr(), self.logits.data_ptr(), ops.scratch_epoch())

    def _run_decode_graph(self, step: StepContext) -> torch.Tensor:
        """A step in which every request brings one token and wants its logits has a fixed shape
        for a given number of requests: its launches are captured once and replayed.  The first
        step of a shape runs directly (it also sizes workspace and scratch), the second is
        captured, later ones replay.  The metadata copy and the sampling stay outside the graph."""
        from ..csrc import ops
        key = (step.n_reqs, step.split_len, tuple(sorted(step.shapes.items())))
        sig = self._buffers_signature()
        if sig != self._graph_sig:
            self.graphs.clear()             # a buffer moved: recorded addresses are stale
            self._graph_seen.clear()
            self._graph_sig = sig
        entry = self.graphs.get(key)
        if entry is None:
            if self._graph_seen.get(key, 0) < 1:
                self._graph_seen[key] = 1
                self.ws.reset()
                out = self.model.forward(step, self.views, self.ws, self.logits)
                after = self._buffers_signature()
                if after != self._graph_sig:
                    # This run moved a buffer (a scratch area grew): every graph captured before holds the
                    # old address, and the old memory goes back to the driver at the next capture
                    # (torch.cuda.graph empties the allocator's cache first).  They are dropped, not kept.
                    self.graphs.clear()
                    self._graph_seen = {key: 1}
                    self._graph_sig = after
                return out
            graph = torch.cuda.CUDAGraph()
            self.ws.reset()
            self.ws.frozen = True
            before = ops.launch_count()
            try:
                with torch.cuda.graph(graph):
                    self.model.forward(step, self.views, self.ws, self.logits)
            finally:
                self.ws.frozen = False
            captured = ops.launch_count() - before
            ops.add_launches(-captured)     # recorded, not run
            entry = (graph, captured)
            self.graphs[key] = entry
            while len(self.graphs) > MAX_CAPTURED_STEPS:           # the least recently replayed goes
                oldest = next(iter(self.graphs))
                del self.graphs[oldest]
                self._graph_seen.pop(oldest, None)
        else:
            self.graphs[key] = self.graphs.pop(key)                # most recently used last
        graph, captured = entry
        graph.replay()
        ops.add_launches(captured)
        return self.logits[: step.n_logit_rows]

    def _prepare(self, entries: List[StepEntry], ids_on_device: bool = False) -> StepContext:
        if not entries:
            raise StepError("a step needs at least one entry")
        r = len(entries)
        if r > self.max_seqs:
            raise StepError(f"{r} requests in one step; max_num_seqs is {self.max_seqs}")
        seen = set()
        q_lens, ctx_lens, slots = [], [], []
        vocab = self.model.vocab
        for e in entries:
            if e.req_id in seen:
                raise StepError(f"request {e.req_id!r} appears twice in one step")
            seen.add(e.req_id)
            if e.req_id not in self.cache.requests:
                raise StepError(f"request {e.req_id!r} is not live; add it to the cache manager first")
            if len(e.tokens) == 0:
                raise StepError(f"request {e.req_id!r} brings no tokens")
            have = self.cache.num_tokens(e.req_id)
            if have + len(e.tokens) > self.max_model_len:
                raise StepError(f"request {e.req_id!r} would hold {have + len(e.tokens)} tokens; "
                                f"max_model_len is {self.max_model_len}")
            if have + len(e.tokens) > self.model.spec.max_position_embeddings:
                raise StepError(f"request {e.req_id!r} would pass max_position_embeddings "
                                f"({self.model.spec.max_position_embeddings})")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise StepError(f"request {e.req_id!r}: wanted place {w} outside its {len(e.tokens)} tokens")
            q_lens.append(len(e.tokens))
            ctx_lens.append(have)
            slots.append(self.cache.slot(e.req_id))
        n = sum(q_lens)
        if n > self.max_tokens:
            raise StepError(f"{n} tokens in one step; max_num_batched_tokens is {self.max_tokens}")
        m = sum(len(e.want) for e in entries)
        for e in entries:
            self.cache.reserve(e.req_id, len(e.tokens))
        if m > self.logits.shape[0]:
            self.logits = torch.empty((m, vocab), dtype=torch.float32, device=self.device)

        # ---- pack the metadata into the pinned buffer, one section after another
        host = HostStep(q_lens, ctx_lens, self.cache.page_size)
        extra = {name: np.ascontiguousarray(b(host), dtype=np.int32) for name, b in self.array_builders.items()}
        total = self._meta_ints(n, r, m) + sum(_align(a.size) for a in extra.values())
        if total > self.meta_host.numel():
            torch.cuda.current_stream().synchronize()
            self.meta_host = torch.empty(total, dtype=torch.int32, pin_memory=True)
            self.meta_dev = torch.empty(total, dtype=torch.int32, device=self.device)
        if self._copy_pending:
            # the pinned buffer is written again only after its last copy has run
            self._copy_done.synchronize()
        hb = self.meta_host.numpy()
        off = 0
        sections = {}

        def section(name, count):
            nonlocal off
            sections[name] = (off, count)
            off += _align(count)
            return hb[sections[name][0]: sections[name][0] + count]

        tok = section("token_ids", n)
        pos = section("positions", n)
        rot = section("req_of_token", n)
        qs = section("q_start", r + 1)
        cl = section("ctx_lens", r)
        sl = section("state_slots", r)
        lr = section("logit_rows", m)
        decode_only = max(q_lens) == 1
        if decode_only:
            # one token per request: every section is a whole-array assignment
            if ids_on_device:
                tok[:] = 0
            else:
                tok[:] = [e.tokens[0] for e in entries]
                if tok.min() < 0 or tok.max() >= vocab:
                    raise StepError(f"a token id lies outside the vocabulary of {vocab}")
            pos[:] = ctx_lens
            rot[:] = np.arange(r, dtype=np.int32)
            qs[:] = np.arange(r + 1, dtype=np.int32)
            mi = 0
            for i, e in enumerate(entries):
                for w in e.want:
                    lr[mi] = i + w
                    mi += 1
        else:
            t0 = 0
            mi = 0
            qs[0] = 0
            for i, e in enumerate(entries):
                ql = q_lens[i]
                ids = np.asarray(e.tokens, dtype=np.int64)
                if ids.min() < 0 or ids.max() >= vocab:
                    raise StepError(f"request {e.req_id!r}: token id outside the vocabulary of {vocab}")
                tok[t0: t0 + ql] = ids
                pos[t0: t0 + ql] = np.arange(ctx_lens[i], ctx_lens[i] + ql)
                rot[t0: t0 + ql] = i
                for w in e.want:
                    lr[mi] = t0 + w
                    mi += 1
                t0 += ql
                qs[i + 1] = t0
        cl[:] = ctx_lens
        sl[:] = slots
        for g in range(self.n_groups):
            # rows of the manager's table array, picked by the requests' slots in one go
            bt = section(f"block_table{g}", r * self.max_blocks).reshape(r, self.max_blocks)
            np.take(self.cache.table_rows(g, self.max_blocks)[:, : self.max_blocks], slots, axis=0, out=bt)
        for name, arr in extra.items():
            section("x:" + name, arr.size)[:] = arr.ravel()
        self.meta_dev[:off].copy_(self.meta_host[:off], non_blocking=True)
        self._copy_done.record()
        self._copy_pending = True
        self.last_meta_bytes = off * 4

        def dev(name, shape=None):
            o, c = sections[name]
            t = self.meta_dev[o: o + c]
            return t if shape is None else t.view(*shape)

        return StepContext(
            n_tokens=n, n_reqs=r, token_ids=dev("token_ids"), positions=dev("positions"),
            req_of_token=dev("req_of_token"), q_start=dev("q_start"), ctx_lens=dev("ctx_lens"),
            block_tables=[dev(f"block_table{g}", (r, self.max_blocks)) for g in range(self.n_groups)],
            state_slots=dev("state_slots"), logit_rows=dev("logit_rows"), n_logit_rows=m,
            h_q_start=[int(x) for x in qs], h_ctx_lens=list(ctx_lens), h_state_slots=list(slots),
            decode_only=decode_only, max_q_len=max(q_lens),
            max_total_len=max(c + q for c, q in zip(ctx_lens, q_lens)),
            split_len=max(256, 1 << (max(c + q for c, q in zip(ctx_lens, q_lens)) - 1).bit_length()),
            extras={name: dev("x:" + name, arr.shape) for name, arr in extra.items()}, shapes=dict(host.shapes))
