"""Arrangements of a layer's parts around the residual stream.

``pre_norm`` is the reference's decoder layer (src/decoder_layer.py:34-54):
``h = h + mixer(norm(h)); h = h + feed_forward(norm(h))``.  The adds are fused into the norm
that follows them, so a block leaves its last product pending in ``hidden.delta``.
"""
from __future__ import annotations

from .base import HiddenState
from .registry import register_part


@register_part("block", "pre_norm")
class PreNormBlock:
    def __init__(self, mixer, feed_forward, norms, params=None) -> None:
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norm_mixer = norms["mixer"]
        self.norm_feed_forward = norms["feed_forward"]

    def forward(self, hidden: HiddenState, ctx, cache) -> None:
        T = ctx.num_tokens
        ws = ctx.workspace
        normed = ws.get("block.normed", (ws.max_tokens, hidden.resid.shape[1]), self.mixer.dtype)
        self.norm_mixer.forward(hidden.resid, hidden.delta, normed, T)
        # A part may add its product into the residual stream itself and return None.
        ctx.residual = hidden.resid
        mixed = self.mixer.forward(normed, ctx, cache)
        self.norm_feed_forward.forward(hidden.resid, mixed, normed, T)
        hidden.delta = self.feed_forward.forward(normed, ctx)
        ctx.residual = None
