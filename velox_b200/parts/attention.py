"""Attention mixer over the paged KV cache.

One forward is: fused q/k/v projection (+bias) -> position encoding on q and k, k and v written
to the cache -> attention of the step's rows over the cache -> output projection
(src/self_attention.py:48-90 of the reference).  A step's tokens attend to themselves through
the cache: the write comes first.  Whether a row belongs to a prompt portion or is a single
decoded token makes no difference here; the step's work layout decides which kernel family
runs which rows.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..ops import kernels
from ..ops.linear import linear, qkv_rope_linear, use_tensor_core_kernel
from .base import CacheNeeds, Mixer, PagedCacheSpec
from .registry import register_part

# VELOX_B200_NO_ROPE_FUSION=1 always rotates in a kernel of its own (for bisecting).
_FUSE_ROPE = os.environ.get("VELOX_B200_NO_ROPE_FUSION") != "1"


@register_part("mixer", "attention")
class Attention(Mixer):
    def __init__(self, params, weights, dtype, device, position=None) -> None:
        super().__init__(params, weights, dtype, device)
        self.hidden_size = int(params["hidden_size"])
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.window: Optional[int] = params.get("window")
        self.softmax_scale = float(params["softmax_scale"])
        if self.num_heads % self.num_kv_heads != 0:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.head_dim % 16 != 0 or not 16 <= self.head_dim <= 256:
            raise ValueError(
                f"head_dim={self.head_dim} is not supported by the attention kernels "
                "(a multiple of 16 between 16 and 256)"
            )
        if position is None:
            raise ValueError("the attention mixer needs a position encoding part ('none' for none)")
        self.position = position
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.qkv_width = self.q_size + 2 * self.kv_size
        self.w_qkv = self.expect("qkv.weight", (self.qkv_width, self.hidden_size))
        self.b_qkv = None
        self.b_qkv_lowp = None
        if params.get("qkv_bias", False):
            self.b_qkv = self.expect("qkv.bias", (self.qkv_width,))
            if dtype != torch.float32:
                self.b_qkv_lowp = self.b_qkv.to(dtype)
        self.w_out = self.expect("out.weight", (self.hidden_size, self.q_size))
        # Compile (or find) the kernels for this head size now, not in the first step.
        kernels.attention_lib(self.head_dim)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(paged=PagedCacheSpec(self.num_kv_heads, self.head_dim, self.window))

    def attention_signature(self):
        return (self.num_kv_heads, self.num_heads // self.num_kv_heads, self.window, self.head_dim)

    # The input is used by the QKV projection only, which can make the norm itself.
    accepts_pending_norm = True
    # Rows of tokens that belong to no sequence (padding of a rounded step) pass through like any
    # other row and are looked at by nobody.
    takes_padded_steps = True

    def forward(self, x, ctx, cache):
        T = ctx.num_tokens
        ws = ctx.workspace
        qkv = ws.get("attention.qkv", (ws.max_tokens, self.qkv_width), self.dtype)
        group = ctx.groups[cache.group]
        k_cache, v_cache = (None, None) if cache.read_only else (cache.k, cache.v)
        # Projection, rotation and cache write in one kernel, where the position encoding
        # offers its tables and the kernel takes the shape (it says no otherwise).
        tables = None
        if _FUSE_ROPE:
            tables = getattr(self.position, "full_rotation_tables", lambda: None)()
        if tables is None or not qkv_rope_linear(
                x, self.w_qkv, self.b_qkv, qkv, T, ctx.status, ctx.positions, tables[0], tables[1],
                group.slot_mapping, k_cache, v_cache, self.num_heads, self.num_kv_heads):
            linear(x, self.w_qkv, self.b_qkv, qkv, T, self.b_qkv_lowp, status=ctx.status)
            self.position.rotate_and_store(qkv, ctx, group.slot_mapping, k_cache, v_cache,
                                           self.num_heads, self.num_kv_heads)

        attn = ws.get("attention.out", (ws.max_tokens, self.q_size), self.dtype)
        plan = ctx.attention_plan(cache.group, self.attention_signature())
        for kind, items, count in plan.launches:
            kernels.attention(
                kind, qkv, attn, cache.k, cache.v, group.block_tables, ctx.q_start, ctx.q_len,
                ctx.kv_len, items, count, plan.partial_o, plan.partial_lse, self.num_heads,
                self.num_kv_heads, self.head_dim, self.window, self.softmax_scale,
                merge_items=plan.merge_items, split_counters=plan.split_counters,
                status=ctx.status,
                cluster=(plan.cluster if kind == kernels.ATTN_BF16_NARROW else
                         getattr(plan, "tc_ctas_per_sm", 1) if kind == kernels.ATTN_BF16_TC else 1),
                layout_checked=getattr(plan, "checked", False),
            )
        if hasattr(plan, "checked"):
            plan.checked = True
        if plan.num_merges and plan.split_counters is None:
            kernels.attention_merge(
                attn, ctx.q_start, plan.merge_items, plan.num_merges, plan.partial_o,
                plan.partial_lse, self.num_heads, self.num_kv_heads, self.head_dim,
                max_rows=plan.merge_rows,
            )

        if ctx.residual is not None and use_tensor_core_kernel(attn, self.w_out, T):
            # Few tokens: the projection is added straight into the float32 residual stream.
            mirror = getattr(ctx, "residual_mirror", None)
            linear(attn, self.w_out, None, ctx.residual, T, status=ctx.status, accumulate=True, mirror=mirror)
            if mirror is not None:
                ctx.residual_mirror_written = True
            return None
        out = ws.get("mixer.out", (ws.max_tokens, self.hidden_size), self.dtype)
        linear(attn, self.w_out, None, out, T, status=ctx.status)
        return out
