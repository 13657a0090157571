"""Arrangements of a layer's parts.

"prenorm":  x += mixer(norm_a(x));  x += feed_forward(norm_b(x))
(src/model/qwen.cpp:300-318).  Each addition is carried as a pending ``delta``
and performed, in float, inside the norm kernel that reads the sum next.
"""
from __future__ import annotations

from .base import Block, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    def forward(self, residual, delta, has_delta, step, cache, writes_cache, ws):
        mark = ws.mark()
        n, hidden = residual.shape
        h = ws.take((n, hidden), delta.dtype)
        self.mixer_norm.forward(residual, delta if has_delta else None, h)
        mixed = ws.take((n, hidden), delta.dtype)
        self.mixer.forward(h, mixed, step, cache, writes_cache, ws)
        self.feed_forward_norm.forward(residual, mixed, h)
        self.feed_forward.forward(h, delta, step, ws)
        ws.release(mark)
        return True
