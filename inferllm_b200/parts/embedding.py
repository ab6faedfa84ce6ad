"""Token embedding and output head.

Embedding: `x[t] = W[id[t]]` (src/kern/naive/naive.cpp:43-54; `EmbdModule`,
src/core/graph.cpp:143-151), written as the float32 residual stream.
Head: `logits = y . W_out^T` in float32 (src/core/op.cpp:230-247 computes it for the last row
only and not at all on prefill, src/core/graph.cpp:132-141; here for the rows the caller
wants).  A tied head uses the embedding table (the reference has no tying).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part, ResidualStream, TensorDecl


class Embedding(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.vocab, self.hidden))}

    def load(self, tensors):
        self.weight = tensors["weight"].to(self.rt.dtype).contiguous()

    def forward(self, ids, ctx) -> ResidualStream:
        return ResidualStream(ops.embedding(ids, self.weight, ctx.err))


class LMHead(Part):
    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])
        self.tied = bool(spec.get("tied", False))
        self.weight = None

    def tensors(self):
        return {} if self.tied else {"weight": TensorDecl((self.vocab, self.hidden))}

    def load(self, tensors):
        if not self.tied:
            self.weight = tensors["weight"].to(self.rt.dtype).contiguous()

    def tie(self, embedding: Embedding):
        self.weight = embedding.weight

    def forward(self, y):
        return ops.linear(y, self.weight, out_dtype=torch.float32)
