"""Position encodings applied to q and k inside an attention mixer.

``rotary_half`` is the reference's RoPE: float32 tables ``angle[p, i] = (p / factor) *
theta^(-2i/R)`` (src/rope.py:45-56) and the rotate-half form ``lo' = lo*cos - hi*sin``,
``hi' = lo*sin + hi*cos`` on the two halves of the first R dims of every head
(src/rope_inplace.py:25-47).  ``none`` rotates nothing.  Both write k and v into the paged
cache in the same kernel that rotates.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from .base import PositionEncoding
from .registry import register_part


@register_part("position", "rotary_half")
class RotaryHalf(PositionEncoding):
    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        self.scaling_factor = float(params.get("scaling_factor", 1.0))
        self.max_position = int(params["max_position"])
        if self.rotary_dim % 2 != 0 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(
                f"rotary_dim={self.rotary_dim} must be even and within head_dim={self.head_dim}"
            )
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        inv_freq = 1.0 / (self.theta ** exponent)
        positions = torch.arange(self.max_position, dtype=torch.float32)
        if self.scaling_factor != 1.0:
            positions = positions / self.scaling_factor
        angles = torch.outer(positions, inv_freq)
        self.cos = angles.cos().to(device).contiguous()
        self.sin = angles.sin().to(device).contiguous()

    def rotate_and_store(self, qkv, ctx, slots, k_cache, v_cache, num_heads, num_kv_heads):
        kernels.rope_cache_write(
            qkv, ctx.positions, self.cos, self.sin, slots, k_cache, v_cache, ctx.num_tokens,
            num_heads, num_kv_heads, self.head_dim, self.rotary_dim, ctx.status,
        )

    def full_rotation_tables(self):
        """(cos, sin) [max_position, head_dim / 2] when every dim of a head rotates, which is
        what a projection that rotates in its epilogue needs; else None."""
        return (self.cos, self.sin) if self.rotary_dim == self.head_dim else None


@register_part("position", "none")
class NoPosition(PositionEncoding):
    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        self.head_dim = int(params["head_dim"])

    def rotate_and_store(self, qkv, ctx, slots, k_cache, v_cache, num_heads, num_kv_heads):
        kernels.rope_cache_write(
            qkv, ctx.positions, None, None, slots, k_cache, v_cache, ctx.num_tokens,
            num_heads, num_kv_heads, self.head_dim, 0, ctx.status,
        )
