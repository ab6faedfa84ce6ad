"""Gated feed-forward (SwiGLU): down( act(gate(h)) * up(h) ), no biases.

The reference's `LlamaFFNModule` (src/core/graph.cpp:57-79) runs w3 (up), w1 (gate), Silu,
Mul, w2 (down) as five operators; silu(x) = x / (1 + exp(-x)) (src/kern/naive/naive.cpp:80-89).
Here gate and up are packed into one [2I, H] matrix at load, row 2i the gate row and row 2i + 1 the
up row of output i, so that one product feeds the activation, and where the package's own kernels run
that product the activation is their epilogue (`kernels.ops.linear_gated`).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, TensorDecl, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        act = spec.get("activation", "silu")
        if act != "silu":
            raise ValueError(f"gated_mlp: activation '{act}' is not supported (only 'silu')")
        self.w_gate_up = None
        self.w_down = None

    def tensors(self):
        return {"gate_proj.weight": TensorDecl((self.inter, self.hidden)),
                "up_proj.weight": TensorDecl((self.inter, self.hidden)),
                "down_proj.weight": TensorDecl((self.hidden, self.inter))}

    def load(self, tensors):
        dt = self.rt.dtype
        self.w_gate_up = torch.stack([tensors["gate_proj.weight"].to(dt), tensors["up_proj.weight"].to(dt)],
                                     dim=1).reshape(2 * self.inter, self.hidden).contiguous()
        self.w_down = tensors["down_proj.weight"].to(dt).contiguous()

    def forward(self, h, ctx):
        return ops.linear(ops.linear_gated(h, self.w_gate_up), self.w_down)

    def forward_deferred(self, h, ctx):
        return ops.linear(ops.linear_gated(h, self.w_gate_up), self.w_down, defer_reduce=True)
