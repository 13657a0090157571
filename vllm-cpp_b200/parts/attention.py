"""Grouped-query self-attention over the paged cache.

q = x Wq^T + bq, k = x Wk^T + bk, v = x Wv^T + bv (bias on q, k, v only in Qwen2:
src/layers/attention.cpp:19-22,74-76); position encoding on q and k
(:79); k and v go to the cache (:84-102); query head h reads kv head
h // (heads / kv_heads) with scale 1/sqrt(d) (:126, src/attention/paged_attention.cu:19);
the result is projected by Wo (:134).

Unlike the reference, q, k and v are one product against [Wq; Wk; Wv]
(concatenated at load), the bias, the rotation and the cache write are one kernel,
a query at position p sees keys 0..p of its own request whatever the batch holds
(the reference has no mask and relies on one token per call), and ``window`` > 0
restricts that to the last ``window`` keys, the query's own included.
"""
from __future__ import annotations

import sys
from typing import Dict

import numpy as np
import torch

from ..config.model_spec import PartSpec
from ..csrc import ops
from .base import (POSITION_ENCODINGS, Mixer, PagedKVSpec, ParamSpec, build_part, register_mixer, workspace_piece)

MAX_HEAD_DIM = 256
_warned_head_dims = set()


@register_mixer("attention")
class PagedAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qkv_bias: bool, out_bias: bool, window: int, position: PartSpec, dtype, device):
        if num_heads <= 0 or num_kv_heads <= 0 or num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} heads cannot share {num_kv_heads} kv heads")
        if head_dim <= 0 or head_dim % 2:
            raise ValueError(f"attention: head_dim {head_dim} must be positive and even")
        if head_dim > MAX_HEAD_DIM:
            raise ValueError(f"attention: head_dim {head_dim} exceeds {MAX_HEAD_DIM}, the largest the kernels take")
        if out_bias:
            raise ValueError("attention: a bias on the output projection is not built")
        if window < 0:
            raise ValueError("attention: window must be 0 (all keys) or positive")
        self.hidden, self.nh, self.nkv, self.d = hidden_size, num_heads, num_kv_heads, head_dim
        self.qkv_bias, self.window = bool(qkv_bias), int(window)
        self.dtype, self.device = dtype, device
        self.position = build_part(POSITION_ENCODINGS, "position encoding", position, dtype=dtype, device=device)
        # 1/sqrtf(d) in float, as src/layers/attention.cpp:126 computes it
        self.scale = float(np.float32(1.0) / np.sqrt(np.float32(head_dim)))
        self.w_qkv = None
        self.b_qkv = None
        self.w_o = None

    # -- tensors
    def param_specs(self) -> Dict[str, ParamSpec]:
        q, kv = self.nh * self.d, self.nkv * self.d
        specs = {"q_proj.weight": ParamSpec((q, self.hidden)),
                 "k_proj.weight": ParamSpec((kv, self.hidden)),
                 "v_proj.weight": ParamSpec((kv, self.hidden)),
                 "o_proj.weight": ParamSpec((self.hidden, q))}
        if self.qkv_bias:
            specs.update({"q_proj.bias": ParamSpec((q,), "bias"),
                          "k_proj.bias": ParamSpec((kv,), "bias"),
                          "v_proj.bias": ParamSpec((kv,), "bias")})
        for name, s in self.position.param_specs().items():
            specs["position." + name] = s
        return specs

    def load_params(self, tensors):
        self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                                tensors["v_proj.weight"]], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"],
                                    tensors["v_proj.bias"]], dim=0).contiguous()
        self.position.load_params({k[len("position."):]: v for k, v in tensors.items()
                                   if k.startswith("position.")})

        if self.dtype == torch.bfloat16 and self.d not in ops.MMA_HEAD_DIMS and self.d not in _warned_head_dims:
            _warned_head_dims.add(self.d)
            print(f"[vllm_cpp_b200] warning: head size {self.d} has no tensor-core attention kernel "
                  f"(those take {ops.MMA_HEAD_DIMS}); bfloat16 attention runs the plain kernel, one warp per "
                  "token and head, many times slower", file=sys.stderr, flush=True)

    # -- cache
    def cache_spec(self):
        return PagedKVSpec(self.nkv, self.d, self.window)

    def workspace_bytes(self, n_tokens, n_reqs):
        q = self.nh * self.d
        return workspace_piece((n_tokens, q + 2 * self.nkv * self.d), self.dtype) + 2 * workspace_piece((n_tokens, q), self.dtype)

    # -- run
    def fuses_norm(self, n_tokens):
        return ops.linear_fuses_norm(n_tokens, self.w_qkv) and ops.linear_fuses_norm(n_tokens, self.w_o)

    def forward(self, x, out, step, cache, writes_cache, ws, x_scale=None, fuse=None):
        n = x.shape[0]
        mark = ws.mark()
        qkv = ws.take((n, (self.nh + 2 * self.nkv) * self.d), self.dtype)
        ops.linear(x, self.w_qkv, qkv, x_scale=x_scale)
        q = ws.take((n, self.nh * self.d), self.dtype)
        block_table = step.block_tables[cache.group]
        fused = self.position.fused()
        bias = self.b_qkv
        if fused is None:
            # An encoding the fused kernel does not know: bias first, then the
            # encoding's own code on q and k, then the plain copy into the cache.
            if bias is not None:
                ops.add_bias(qkv, bias)
                bias = None
            q3 = qkv[:, : self.nh * self.d].unflatten(1, (self.nh, self.d))
            k3 = qkv[:, self.nh * self.d: (self.nh + self.nkv) * self.d].unflatten(1, (self.nkv, self.d))
            self.position.apply(q3, k3, step.positions)
            fused = {"rotary_dim": 0, "pairing": 0, "denom": None}
        ops.rope_cache_write(qkv, bias, step.positions, step.req_of_token, block_table, fused["denom"], q,
                             cache.pages, num_heads=self.nh, num_kv_heads=self.nkv, head_dim=self.d,
                             rotary_dim=fused["rotary_dim"], pairing=fused["pairing"],
                             page_size=cache.page_size, write_kv=writes_cache)
        attn = ws.take((n, self.nh * self.d), self.dtype)
        self.attend(q, attn, step, cache, block_table)
        ops.linear(attn, self.w_o, out, fuse=fuse)
        ws.release(mark)

    # -- work lists and kernel choice
    def _tensor_core_path(self) -> bool:
        return self.dtype == torch.bfloat16 and self.d in ops.MMA_HEAD_DIMS


    def step_arrays(self):
        """What the kernels need per step beyond the common arrays, built on the host from the step's
        lengths.  The prefill kernel's work list: for every request that brings tokens, its tiles of
        packed rows (token x head in group, ops.TC_ATTENTION_TILE_ROWS of them), as [2, n_tiles] =
        (request index, first row).  The decode kernel's split length: see ``splits`` below."""
        if not self._tensor_core_path():
            return {}
        group = self.nh // self.nkv

        def tiles(host):
            if all(q == 1 for q in host.q_lens):
                return np.zeros((2, 0), dtype=np.int32)         # decode-only steps use the split-KV kernel
            rows = ops.TC_ATTENTION_TILE_ROWS
            req, row0, keys = [], [], []
            for r, (q, ctx) in enumerate(zip(host.q_lens, host.ctx_lens)):
                for k in range(-(-q * group // rows)):
                    req.append(r)
                    row0.append(k * rows)
                    keys.append(ctx + min(q, ((k + 1) * rows + group - 1) // group))   # keys its last row sees
            # CTAs start in list order: the tiles with the most keys go first, so that the short
            # ones fill the tail instead of the other way round (causal work is triangular)
            order = np.argsort(-np.asarray(keys), kind="stable")
            return np.array([req, row0], dtype=np.int32)[:, order]

        def splits(host):
            """Decode-only steps: [most key tiles a split may have], and the grid's columns as a launch
            shape.  A request gets as many splits as its context needs under that bound, so one with a
            long context gets more CTAs than one with a short context.  The bound is the smallest with
            which the splits of all requests fit decode_slots() (one round of CTAs; a second would
            double the time).  Equal contexts come out as before: all requests in equal parts."""
            if any(q != 1 for q in host.q_lens):
                return np.zeros(1, dtype=np.int32)
            tile, most = ops.DECODE_KEY_TILE, ops.DECODE_MAX_SPLITS
            hi = np.asarray(host.ctx_lens, dtype=np.int64) + 1
            lo = np.maximum(0, hi - self.window) if self.window > 0 else np.zeros_like(hi)
            n = -(-hi // tile) - lo // tile                     # key tiles of every request
            slots = self.decode_slots(len(n))
            low, high = max(1, -(-int(n.sum()) // slots)), int(n.max())
            while low < high:                                   # smallest count whose splits fit the slots
                mid = (low + high) // 2
                if int((-(-n // mid)).sum()) <= slots:
                    high = mid
                else:
                    low = mid + 1
            longest = int(n.max())
            # with few requests the slots would allow splits of one or two tiles, but below four tiles a
            # split's start, its partials and a longer merge cost more than its share of the keys: at least
            # four tiles a split, unless that leaves the longest request fewer than eight splits
            per = max(low, -(-longest // most), min(4, -(-longest // 8)))
            need = -(-longest // per)
            # the grid's columns: the next size of a short ladder, so that few shapes are captured and at
            # most a quarter of a request's CTAs find nothing to do (they cost a launch each)
            host.shapes[self._splits_key()] = next(g for g in self.SPLIT_GRIDS if g >= need)
            return np.array([per], dtype=np.int32)

        return {f"attn_tiles_g{group}": tiles, self._splits_key(): splits}

    SPLIT_GRIDS = (1, 2, 3, 4, 5, 6, 8, 10, 12, 16, 20, 24, 32)

    def decode_slots(self, n_reqs: int) -> int:
        """Splits per kv head that a decode step may have in all: seven eighths of the places the device has
        for the kernel's CTAs (two per SM).  Filling every place was measured slower: the CTAs of the
        kernels before and after share the SMs, and a CTA that finds no place waits for a second round."""
        return max(n_reqs, (2 * ops.sm_count() * 7 // 8) // self.nkv)

    def reserve(self, n_tokens, n_reqs, device):
        if self._tensor_core_path():
            most = n_reqs * self.nh * ops.DECODE_MAX_SPLITS
            ops.scratch("attn_part_o", most * self.d, device)
            ops.scratch("attn_part_ml", most * 2, device)
            ops.zeroed_ints("attn_tickets", n_reqs * self.nkv, device)

    def _splits_key(self):
        return f"attn_splits_kv{self.nkv}_w{self.window}"

    def attend(self, q, attn, step, cache, block_table):
        if self._tensor_core_path():
            kw = dict(num_heads=self.nh, num_kv_heads=self.nkv, head_dim=self.d, page_size=cache.page_size,
                      window=self.window, scale=self.scale)
            if step.decode_only:
                nsplit = step.shapes.get(self._splits_key())
                split_tiles = step.extras.get(self._splits_key())
                if nsplit is None:
                    # a step without the builder's arrays: every request in equal parts, as many as fill
                    # the device once, from the longest context's power-of-two bucket
                    longest = step.split_len or step.max_total_len
                    if self.window > 0:
                        longest = min(longest, self.window + 64)
                    nsplit = max(1, min(-(-longest // 64), 2 * ops.sm_count() // (step.n_reqs * self.nkv),
                                        ops.DECODE_MAX_SPLITS))
                    split_tiles = None
                part_o = part_ml = counters = None
                if nsplit > 1:
                    need = step.n_reqs * self.nh * nsplit
                    part_o = ops.scratch("attn_part_o", need * self.d, q.device)
                    part_ml = ops.scratch("attn_part_ml", need * 2, q.device)
                    counters = ops.zeroed_ints("attn_tickets", step.n_reqs * self.nkv, q.device)
                ops.attention_decode_mma(q, cache.pages, attn, step.q_start, step.ctx_lens, block_table, None,
                                         step.n_reqs, nsplit, part_o, part_ml, counters, split_tiles=split_tiles, **kw)
            else:
                tiles = step.extras[f"attn_tiles_g{self.nh // self.nkv}"]
                ops.attention_prefill_tc(q, cache.pages, attn, step.q_start, step.ctx_lens, block_table, tiles[0], tiles[1], **kw)
            return
        ops.attention_simt(q, cache.pages, attn, step.positions, step.req_of_token, block_table,
                           num_heads=self.nh, num_kv_heads=self.nkv, head_dim=self.d,
                           page_size=cache.page_size, window=self.window, scale=self.scale)
