"""Matrix products of the model: ``y = x @ W.T + b`` with W stored [out, in].

float32: this package's own FP32-pipe kernel, always (no TF32, no tensor cores): it is the
true 32-bit path and sums every output element in a fixed order.

bfloat16: a library GEMM (cuBLAS through torch), which is what the reference engine uses for
every projection (``nn.Linear``, src/self_attention.py:32-33, src/mlp.py:9-10,
src/transformer.py:60).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import kernels


def linear(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias_f32: Optional[torch.Tensor],
    out: torch.Tensor,
    num_rows: int,
    bias_lowp: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """out[:num_rows] = x[:num_rows] @ weight.T (+ bias).  Returns ``out``."""
    if num_rows == 0:
        return out
    if weight.dtype == torch.float32:
        kernels.gemm_f32(x, weight, bias_f32, out, num_rows)
        return out
    if weight.dtype != torch.bfloat16:
        raise TypeError(f"linear: weights must be float32 or bfloat16, got {weight.dtype}")
    xs, os_ = x[:num_rows], out[:num_rows]
    if bias_f32 is not None:
        if bias_lowp is None:
            raise ValueError("the bfloat16 library GEMM needs the bias in bfloat16 too")
        torch.addmm(bias_lowp, xs, weight.t(), out=os_)
    else:
        torch.mm(xs, weight.t(), out=os_)
    return out
