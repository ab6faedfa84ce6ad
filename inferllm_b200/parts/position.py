"""Position encodings of the attention mixer.

"rope_half" is the reference's `RotMode::ModelRotHalf` (src/kern/naive/naive.cpp:389-414):
pair (j, j + rot/2) of every Q and K head is rotated by the angle `p * theta^(-2j/rot)`.
The reference computes the trigonometry per element (in double on the CPU, with
powf/sinf/cosf on the GPU, src/kern/gpu/kernel_gpu.cu:343-371); here a table
[position, rot/2, (cos, sin)] is computed once in float64 and stored in float32, and the
rotation is done in float32 inside the kernel that also writes K and V into the cache.
theta (fixed to 10000 in the reference) and rot_dim are parameters.

"none" encodes nothing and only stores K and V.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import PositionEncoding, register_position


@register_position("rope_half")
class RopeHalf(PositionEncoding):
    takes_partials = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.head_dim = int(spec["head_dim"])
        self.rot_dim = int(spec.get("rot_dim", self.head_dim))
        self.theta = float(spec["theta"])
        self.max_positions = int(spec["max_positions"])
        if self.rot_dim % 2 or not 0 < self.rot_dim <= self.head_dim:
            raise ValueError(f"rope_half: rot_dim {self.rot_dim} must be even and in (0, head_dim]")
        self.table = None

    def prepare(self):
        half = self.rot_dim // 2
        j = torch.arange(half, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * j / self.rot_dim)
        ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * inv[None, :]
        table = torch.stack((torch.cos(ang), torch.sin(ang)), dim=-1).to(torch.float32)
        self.table = table.contiguous().to(self.rt.device)

    def rotation_table(self):
        return (self.table, self.rot_dim)

    def encode_and_store(self, qkv, geometry, ctx, kv):
        n_heads, n_kv_heads, head_dim = geometry
        return ops.rope_kv_write(qkv, self.table, self.rot_dim, ctx.token_pos, ctx.token_seq,
                                 kv.block_table, kv.k if kv.writes else None, kv.v if kv.writes else None,
                                 n_heads, n_kv_heads, head_dim, kv.page_size, kv.writes, ctx.err)


@register_position("none")
class NoPosition(PositionEncoding):
    takes_partials = True

    def rotation_table(self):
        return (None, 0)

    def encode_and_store(self, qkv, geometry, ctx, kv):
        n_heads, n_kv_heads, head_dim = geometry
        if kv.writes:
            return ops.rope_kv_write(qkv, None, 0, ctx.token_pos, ctx.token_seq, kv.block_table, kv.k, kv.v,
                                     n_heads, n_kv_heads, head_dim, kv.page_size, True, ctx.err)
        return qkv
