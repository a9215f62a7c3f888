"""Dense feed-forward parts.  ``swiglu`` is the reference's MLP: ``down(silu(gate(x)) * up(x))``
with gate and up fused into one matrix whose first half is gate, and no biases
(src/mlp.py:9-15).  SiLU and the product are computed in float32 and rounded once (the reference
rounds to the model dtype between the two)."""
from __future__ import annotations

from ..ops import kernels
from ..ops.linear import linear, swiglu_linear, use_tensor_core_kernel
from .base import FeedForward
from .registry import register_part


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

    def forward(self, x, ctx):
        T = ctx.num_tokens
        ws = ctx.workspace
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
