"""Gated feed-forward (SwiGLU): down( act(gate(h)) * up(h) ), no biases.

The reference's `LlamaFFNModule` (src/core/graph.cpp:57-79) runs w3 (up), w1 (gate), Silu,
Mul, w2 (down) as five operators; silu(x) = x / (1 + exp(-x)) (src/kern/naive/naive.cpp:80-89).
Here gate and up are stacked into one [2I, H] matrix at load, so one product feeds the
activation kernel.
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
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"].to(dt),
                                    tensors["up_proj.weight"].to(dt)], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].to(dt).contiguous()

    def forward(self, h, ctx):
        gu = ops.linear(h, self.w_gate_up, defer_reduce=True)     # the activation kernel adds K slices up
        return ops.linear(ops.swiglu(gu), self.w_down)

    def forward_deferred(self, h, ctx):
        gu = ops.linear(h, self.w_gate_up, defer_reduce=True)
        return ops.linear(ops.swiglu(gu), self.w_down, defer_reduce=True)
