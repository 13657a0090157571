"""Arrangements of a layer's parts.

"prenorm":  x += mixer(norm_a(x));  x += feed_forward(norm_b(x))
(src/model/qwen.cpp:300-318).  Each addition is carried as a pending ``delta``
and performed, in float, inside the norm kernel that reads the sum next.

Where the parts on both sides of a norm say they can (``fuses_norm``) and the norm can be
split (``Norm.split``), no norm kernel runs: the product that ends the branch before the
norm adds its result to the residual stream, multiplies by the gain and leaves the rows'
sums of squares, and the product after the norm applies the factor (ops.ResidualNorm,
ops.RowScale).  That holds for the norm inside the layer and for the one the next layer
starts with.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Block, register_block, workspace_piece


@register_block("prenorm")
class PreNormBlock(Block):
    def accepts_prenormed(self, n_tokens):
        return self.mixer_norm.split() if self.mixer.fuses_norm(n_tokens) else None

    def workspace_bytes(self, n_tokens, n_reqs, hidden, dtype):
        own = 2 * workspace_piece((n_tokens, hidden), dtype) \
            + workspace_piece((ops.sumsq_parts(hidden), n_tokens), torch.float32)
        return own + super().workspace_bytes(n_tokens, n_reqs, hidden, dtype)

    def forward(self, residual, delta, pending, step, cache, writes_cache, ws, next_block=None, carry=None):
        mark = ws.mark()
        n, hidden = residual.shape
        h = ws.take((n, hidden), delta.dtype)
        mixed = ws.take((n, hidden), delta.dtype)
        if isinstance(pending, ops.RowScale):
            x, scale_kw = delta, {"x_scale": pending}
        else:
            self.mixer_norm.forward(residual, delta if pending else None, h)
            x, scale_kw = h, {}
        inner = self.feed_forward_norm.split()
        if inner is None or carry is None or not (self.mixer.fuses_norm(n) and self.feed_forward.fuses_norm(n)):
            self.mixer.forward(x, mixed, step, cache, writes_cache, ws, **scale_kw)
            self.feed_forward_norm.forward(residual, mixed, h)
            self.feed_forward.forward(h, delta, step, ws)
            ws.release(mark)
            return True
        # the mixer's last product ends its branch: residual += ..., mixed = residual * gain
        sumsq = ws.take((ops.sumsq_parts(hidden), n), torch.float32)
        ends = ops.ResidualNorm(residual, inner[0], sumsq, inner[1])
        self.mixer.forward(x, mixed, step, cache, writes_cache, ws, fuse=ends, **scale_kw)
        after = next_block.accepts_prenormed(n) if next_block is not None else None
        if after is None:
            self.feed_forward.forward(mixed, delta, step, ws, x_scale=ends.scale())
            ws.release(mark)
            return True
        # the feed-forward's last product does the same for the norm the next layer starts with
        came_in = pending.sumsq.data_ptr() if isinstance(pending, ops.RowScale) else None
        out_sumsq = carry[1] if came_in == carry[0].data_ptr() else carry[0]
        ends_layer = ops.ResidualNorm(residual, after[0], out_sumsq, after[1])
        self.feed_forward.forward(mixed, delta, step, ws, x_scale=ends.scale(), fuse=ends_layer)
        ws.release(mark)
        return ends_layer.scale()
