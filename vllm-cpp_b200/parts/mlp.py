"""Gated feed-forward: down( act(gate(x)) * up(x) ), no biases
(src/layers/mlp.cpp:49-64; silu of src/kernels/activation.cu:8-10).

gate and up are one product against the row-wise concatenation [W_gate; W_up],
made at load; the reference runs them as two.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import FeedForward, ParamSpec, register_feed_forward, workspace_piece


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, activation: str, dtype, device):
        if activation != "silu":
            raise ValueError(f"gated_mlp: activation {activation!r} is not built (only 'silu')")
        self.hidden, self.inter = hidden_size, intermediate_size
        self.dtype, self.device = dtype, device
        self.w_gate_up = None     # [2*inter, hidden]
        self.w_down = None        # [hidden, inter]

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"gate_proj.weight": ParamSpec((self.inter, self.hidden)),
                "up_proj.weight": ParamSpec((self.inter, self.hidden)),
                "down_proj.weight": ParamSpec((self.hidden, self.inter))}

    def load_params(self, tensors):
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def product_weights(self):
        return [(self.w_gate_up, self.inter), (self.w_down, 0)]

    def fuses_norm(self, n_tokens):
        return ops.linear_fuses_norm(n_tokens, self.w_gate_up) and ops.linear_fuses_norm(n_tokens, self.w_down)

    def workspace_bytes(self, n_tokens, n_reqs):
        # the activations, and the gate-and-up product where the activation is a kernel of its own
        return workspace_piece((n_tokens, self.inter), self.dtype) + workspace_piece((n_tokens, 2 * self.inter), self.dtype)

    def forward(self, x, out, step, ws, x_scale=None, fuse=None):
        n = x.shape[0]
        mark = ws.mark()
        act = ws.take((n, self.inter), self.dtype)
        if ops.linear_gated_fuses(n, self.w_gate_up):
            ops.linear_gated(x, self.w_gate_up, act, x_scale=x_scale)       # product and activation in one kernel
        else:
            gate_up = ws.take((n, 2 * self.inter), self.dtype)
            ops.linear(x, self.w_gate_up, gate_up, x_scale=x_scale)
            ops.silu_mul(gate_up, act)
        ops.linear(act, self.w_down, out, fuse=fuse)
        ws.release(mark)
