"""RMSNorm fused with the residual add (the reference's norm: src/rmsnorm.py:20-28; its adds:
src/decoder_layer.py:49,54)."""
from __future__ import annotations

from ..ops import kernels
from .base import Norm, PendingNorm
from .registry import register_part


@register_part("norm", "rms")
class RMSNorm(Norm):
    """``out = v * rsqrt(mean(v^2) + eps) * weight`` with ``v = resid + delta``, in float32."""

    def __init__(self, params, weights, dtype, device) -> None:
        super().__init__(params, weights, dtype, device)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight = self.expect("weight", (self.size,))

    def forward(self, resid, delta, out, num_rows, rows=None, write_resid=True):
        kernels.add_rmsnorm(resid, delta, self.weight, self.eps, out, num_rows, rows, write_resid)
        return out

    def pending(self, resid, out, num_rows):
        return PendingNorm(self, resid, out, num_rows)
