"""RMSNorm with a weight, fused with the residual addition that precedes it.

Formula of the reference (src/kern/naive/naive.cpp:186-207, weight multiply :138-149):
`y = x / sqrt(mean(x^2) + eps) * w`.  The reference fixes eps in code (1e-6 in the layers,
src/graph/llama_like.cpp:77-78; 1e-5 in the head, src/core/graph.h:160-163); here it is a
parameter of the part.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm, TensorDecl, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.size,), "norm")}

    def load(self, tensors):
        w = tensors["weight"]
        # a weight stored in 32-bit stays 32-bit; bfloat16 stays bfloat16 (the kernel takes both)
        if w.dtype not in (torch.float32, torch.bfloat16):
            w = w.to(torch.float32 if self.rt.is_f32 else torch.bfloat16)
        self.weight = w.contiguous()

    def forward(self, stream, rows=None):
        y = ops.add_rmsnorm(stream.x, stream.pending, self.weight, self.eps, self.rt.dtype,
                            rows=rows, write_resid=rows is None)
        if rows is None:
            stream.pending = None
        return y
