"""Dense feed-forward parts.  ``swiglu`` is the reference's MLP: ``down(silu(gate(x)) * up(x))``
with gate and up fused into one matrix whose first half is gate, and no biases
(src/mlp.py:9-15).  SiLU and the product are computed in float32 and rounded once (the reference
rounds to the model dtype between the two)."""
from __future__ import annotations

import os

import torch

from ..ops import kernels
from ..ops.linear import DETERMINISTIC, linear, swiglu_linear, use_tensor_core_kernel
from .base import FeedForward
from .registry import register_part


# VELOX_B200_NO_MLP_FUSION=1 keeps the two projections of a small step as kernels of their own
# (for bisecting; the fused kernel's sum over the inner width has no fixed order).
_FUSE_MLP = os.environ.get("VELOX_B200_NO_MLP_FUSION") != "1" and not DETERMINISTIC


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        self.hidden_size = int(params["hidden_size"])
        self.intermediate_size = int(params["intermediate_size"])
        self.w_gate_up = self.expect("gate_up.weight", (2 * self.intermediate_size, self.hidden_size))
        self.w_down = self.expect("down.weight", (self.hidden_size, self.intermediate_size))

    # The input is used by the gate|up projection only, which can make the norm itself.
    accepts_pending_norm = True
    # Rows of tokens that belong to no sequence (padding of a rounded step) pass through like any
    # other row and are looked at by nobody.
    takes_padded_steps = True

    def _fusable(self, T, ctx) -> bool:
        return (_FUSE_MLP and 0 < T <= kernels.MLP_FUSED_MAX_TOKENS and self.dtype == torch.bfloat16
                and ctx.status is not None and self.hidden_size % 128 == 0 and self.intermediate_size % 64 == 0)

    def wants_residual_mirror(self, T, ctx) -> bool:
        """With few tokens the whole feed-forward is one kernel whose CTAs add their shares into
        the residual stream while others still read their input rows: it reads a copy."""
        return self._fusable(T, ctx)

    def forward(self, x, ctx):
        T = ctx.num_tokens
        ws = ctx.workspace
        if (self._fusable(T, ctx) and ctx.residual is not None and getattr(x, "resid", None) is not None
                and x.resid.data_ptr() != ctx.residual.data_ptr() and x.resid.dtype == torch.float32):
            if kernels.mlp_fused(x.resid, x.weight, x.eps, self.w_gate_up, self.w_down, ctx.residual, T, ctx.status):
                return None
        act = ws.get("swiglu.act", (ws.max_tokens, self.intermediate_size), self.dtype)
        if use_tensor_core_kernel(x, self.w_gate_up, T) and use_tensor_core_kernel(act, self.w_down, T):
            # Few tokens: SiLU(gate) * up in the projection's epilogue, then the down projection
            # added straight into the float32 residual stream.
            swiglu_linear(x, self.w_gate_up, act, T, ctx.status)
            if ctx.residual is not None:
                linear(act, self.w_down, None, ctx.residual, T, status=ctx.status, accumulate=True)
                return None
            out = ws.get("feed_forward.out", (ws.max_tokens, self.hidden_size), self.dtype)
            linear(act, self.w_down, None, out, T, status=ctx.status)
            return out
        gate_up = ws.get("swiglu.gate_up", (ws.max_tokens, 2 * self.intermediate_size), self.dtype)
        linear(x, self.w_gate_up, None, gate_up, T)
        kernels.swiglu(gate_up, act, T)
        out = ws.get("feed_forward.out", (ws.max_tokens, self.hidden_size), self.dtype)
        linear(act, self.w_down, None, out, T)
        return out
