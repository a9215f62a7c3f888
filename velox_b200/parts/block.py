"""Arrangements of a layer's parts around the residual stream.

``pre_norm`` is the reference's decoder layer (src/decoder_layer.py:34-54):
``h = h + mixer(norm(h)); h = h + feed_forward(norm(h))``.  The adds are fused into the norm
that follows them, so a block leaves its last product pending in ``hidden.delta``.
"""
from __future__ import annotations

import os

import torch

from .base import HiddenState
from .registry import register_part

# VELOX_B200_NO_NORM_FUSION=1 runs every norm as a kernel of its own (for bisecting).
_FUSE_NORMS = os.environ.get("VELOX_B200_NO_NORM_FUSION") != "1"


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
        # A part may add its product into the residual stream itself and return None.
        ctx.residual = hidden.resid
        # A feed-forward that adds into the stream while it still reads its input asks for a
        # copy of the rows; a mixer that adds its product itself can write it on the way.
        ctx.residual_mirror = None
        ctx.residual_mirror_written = False
        wants = getattr(self.feed_forward, "wants_residual_mirror", None)
        if wants is not None and wants(T, ctx):
            ctx.residual_mirror = ws.get("block.residual_mirror", (ws.max_tokens, hidden.resid.shape[1]), torch.float32)
        mixed = self.mixer.forward(self._normed(self.norm_mixer, self.mixer, hidden.resid, hidden.delta, normed, T),
                                   ctx, cache)
        source = hidden.resid
        if mixed is None and ctx.residual_mirror is not None and ctx.residual_mirror_written:
            source = ctx.residual_mirror
        hidden.delta = self.feed_forward.forward(
            self._normed(self.norm_feed_forward, self.feed_forward, source, mixed, normed, T), ctx)
        ctx.residual = None
        ctx.residual_mirror = None

    @staticmethod
    def _normed(norm, consumer, resid, delta, out, num_rows):
        """The consumer's input: the norm's output, or, when nothing is waiting to be added and
        the consumer can take it, the norm itself for its first projection to make."""
        if _FUSE_NORMS and delta is None and getattr(consumer, "accepts_pending_norm", False):
            pending = norm.pending(resid, out, num_rows)
            if pending is not None:
                return pending
        norm.forward(resid, delta, out, num_rows)
        return out
