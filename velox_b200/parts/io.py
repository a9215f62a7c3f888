"""The two ends of a model: token embedding and the language-model head
(src/transformer.py:27,44 and 60-68 of the reference)."""
from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import linear, use_tensor_core_kernel
from .base import Part
from .registry import register_part


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    """``resid[t] = table[ids[t]]``, widened to the float32 residual stream."""

    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.table = self.expect("weight", (self.vocab_size, self.hidden_size))

    def forward(self, ids, resid, ctx) -> None:
        # ctx.fed_tokens: the sampler's tokens of the step before, for ids that name one of them.
        kernels.embed(self.table, ids[: ctx.num_tokens], resid, ctx.status, getattr(ctx, "fed_tokens", None))


@register_part("lm_head", "linear_head")
class LinearHead(Part):
    """``logits = x @ W.T`` without bias, returned in float32."""

    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        self.vocab_size = int(params["vocab_size"])
        self.hidden_size = int(params["hidden_size"])
        self.weight = self.expect("weight", (self.vocab_size, self.hidden_size))

    def forward(self, x, num_rows, ctx) -> torch.Tensor:
        ws = ctx.workspace
        logits = ws.get("lm_head.logits", (ws.max_logit_rows, self.vocab_size), torch.float32)
        if self.dtype == torch.float32:
            linear(x, self.weight, None, logits, num_rows)
        elif use_tensor_core_kernel(x, self.weight, num_rows):
            # float32 logits straight from the accumulators
            linear(x, self.weight, None, logits, num_rows, status=ctx.status)
        else:
            low = ws.get("lm_head.logits_lowp", (ws.max_logit_rows, self.vocab_size), self.dtype)
            linear(x, self.weight, None, low, num_rows)
            kernels.cast_bf16_to_f32(low, logits, num_rows * self.vocab_size)
        return logits[:num_rows]
