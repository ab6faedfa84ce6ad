"""Causal self-attention with grouped heads over the paged cache: the mixer of LLaMA.

Order of operations of the reference's `LlamaAttention::execute` (src/core/op.cpp:348-500):
Q, K, V projections without bias; position encoding of Q and of the new K rows; K and V go
into the cache; scores of every query against all cached keys of its sequence, scaled by
1/sqrt(head size) (:488) and masked causally; softmax; weighted values; then the output
projection (`AttentionModule`, src/core/graph.h:106-111).  The reference has separate
[H, H] matrices and one KV head per query head (src/core/op.h:327-332); here the three
matrices are stacked into one [(heads + 2 kv heads) * d, H] at load so that one product
feeds the rotation kernel, and the number of KV heads, the head size and an optional window
are parameters.
"""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from .base import Mixer, PagedKV, TensorDecl, build_part, register_mixer


@register_mixer("attention")
class Attention(Mixer):
    graph_safe = True   # a decode step's launches depend only on the batch size

    @property
    def pad_safe(self) -> bool:
        """Causal attention: tokens behind a sequence's real ones are seen by none of them.  Said
        only for the plain case: no window, and a position encoding that is nothing but the table
        rotation (any other runs code of its own, which is not known to launch the same kernels)."""
        return self.window is None and self.position.rotation_table() is not None

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec["hidden_size"])
        self.n_heads = int(spec["n_heads"])
        self.n_kv_heads = int(spec["n_kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.window = spec.get("window")
        self.scale = float(spec.get("scale") or 1.0 / math.sqrt(self.head_dim))
        if self.n_heads % self.n_kv_heads:
            raise ValueError("attention: n_heads must be a multiple of n_kv_heads")
        self.position = build_part("position", spec["position"], runtime)
        if runtime is not None:
            self.position.prepare()
        self.w_qkv = None
        self.w_o = None

    def tensors(self):
        q, kv = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        return {"q_proj.weight": TensorDecl((q, self.hidden)),
                "k_proj.weight": TensorDecl((kv, self.hidden)),
                "v_proj.weight": TensorDecl((kv, self.hidden)),
                "o_proj.weight": TensorDecl((self.hidden, q))}

    def load(self, tensors):
        dt = self.rt.dtype
        self.w_qkv = torch.cat([tensors["q_proj.weight"].to(dt), tensors["k_proj.weight"].to(dt),
                                tensors["v_proj.weight"].to(dt)], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].to(dt).contiguous()

    def cache_request(self):
        return PagedKV(self.n_kv_heads, self.head_dim, self.window)

    def forward(self, h, ctx, cache, writes):
        return self._run(h, ctx, cache, False)

    def forward_deferred(self, h, ctx, cache, writes):
        return self._run(h, ctx, cache, True)

    def _run(self, h, ctx, cache, defer_output):
        rotation = self.position.rotation_table()
        if (ctx.is_decode and rotation is not None and rotation[1] % 16 == 0
                and ops.attention_decode_ring_supported(h.dtype, self.n_heads, self.n_kv_heads, self.head_dim,
                                                        cache.page_size)):
            # one token per sequence: the attention kernel itself adds up the K slices of the
            # projection, rotates Q and the new K row and writes K and V into the cache
            qkv = ops.linear(h, self.w_qkv, defer_reduce=True)
            o = ops.attention_decode_ring(qkv, cache.k, cache.v, cache.block_table, ctx.token_pos, ctx.token_seq,
                                          self.n_heads, self.n_kv_heads, self.head_dim, cache.page_size,
                                          self.window, self.scale, ctx.max_seq_len,
                                          rope=(rotation[0], rotation[1], cache.writes, ctx.err))
            return ops.linear(o, self.w_o, defer_reduce=defer_output)
        # the packed projection may stay in K slices if the position encoding's kernel adds them up
        qkv = ops.linear(h, self.w_qkv, defer_reduce=self.position.takes_partials)
        geometry = (self.n_heads, self.n_kv_heads, self.head_dim)
        qkv = self.position.encode_and_store(qkv, geometry, ctx, cache)
        o = ops.attention(qkv, cache, ctx, self.n_heads, self.n_kv_heads, self.head_dim,
                          self.window, self.scale)
        return ops.linear(o, self.w_o, defer_reduce=defer_output)
