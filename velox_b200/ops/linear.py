"""Matrix products of the model: ``y = x @ W.T + b`` with W stored [out, in].

float32: this package's own FP32-pipe kernel, always (no TF32, no tensor cores): it is the
true 32-bit path and sums every output element in a fixed order.

bfloat16: the tcgen05/TMA kernel of ``csrc/gemm_bf16.cu`` when the step has few tokens (decode
and short portions: the weight fills the 128-row side of the tensor-core tile and is streamed
once; key ranges are split over CTAs to fill the GPU), a library GEMM (cuBLAS through torch)
for long portions and for inner sizes the TMA tiles cannot take.  The reference engine uses a
library GEMM for every projection (``nn.Linear``, src/self_attention.py:32-33,
src/mlp.py:9-10, src/transformer.py:60 of that project).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Union

import torch

from . import kernels

# Steps with at most this many tokens use the tcgen05 kernel for their projections.
SMALL_STEP_TOKENS = 256
_NUM_SMS = None


def _num_sms() -> int:
    global _NUM_SMS
    if _NUM_SMS is None:
        _NUM_SMS = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _NUM_SMS


@dataclass
class Partials:
    """A product that exists as float32 split sums: the value is ``data[:count].sum(0)``."""

    data: torch.Tensor  # float32 [splits, rows, N]
    count: int


def use_tensor_core_kernel(x: torch.Tensor, weight: torch.Tensor, num_rows: int) -> bool:
    return (
        weight.dtype == torch.bfloat16
        and num_rows <= SMALL_STEP_TOKENS
        and kernels.gemm_bf16_supported(x, weight)
    )


MAX_SPLITS = 16


def choose_splits(out_features: int, in_features: int, num_rows: int, tile: int = 128) -> int:
    """Splits of the inner dimension so that tiles x splits is about the number of SMs, with at
    least two 64-wide blocks per split and at most about 4 MB of split products."""
    tiles = -(-out_features // tile)
    blocks = -(-in_features // 64)
    by_traffic = max(1, (4 << 20) // max(1, num_rows * out_features * 4))
    return max(1, min(_num_sms() // max(tiles, 1), blocks // 2, by_traffic, MAX_SPLITS))


def split_scratch(workspace, out_features: int) -> torch.Tensor:
    """The float32 buffer [MAX_SPLITS, rows, N] that split products of width N are written to."""
    rows = min(workspace.max_tokens, SMALL_STEP_TOKENS)
    return workspace.get(f"linear.partials.{out_features}", (MAX_SPLITS, rows, out_features), torch.float32)


def linear(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias_f32: Optional[torch.Tensor],
    out: torch.Tensor,
    num_rows: int,
    bias_lowp: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """out[:num_rows] = x[:num_rows] @ weight.T (+ bias), in the dtype of ``out``."""
    if num_rows == 0:
        return out
    if weight.dtype == torch.float32:
        kernels.gemm_f32(x, weight, bias_f32, out, num_rows)
        return out
    if weight.dtype != torch.bfloat16:
        raise TypeError(f"linear: weights must be float32 or bfloat16, got {weight.dtype}")
    if status is not None and use_tensor_core_kernel(x, weight, num_rows):
        mode = kernels.GEMM_OUT_F32 if out.dtype == torch.float32 else kernels.GEMM_OUT_BF16
        kernels.gemm_bf16(x, weight, bias_f32, out, mode, num_rows, status)
        return out
    if out.dtype != torch.bfloat16:
        raise TypeError("the library GEMM path writes bfloat16")
    xs, os_ = x[:num_rows], out[:num_rows]
    if bias_f32 is not None:
        if bias_lowp is None:
            raise ValueError("the bfloat16 library GEMM needs the bias in bfloat16 too")
        torch.addmm(bias_lowp, xs, weight.t(), out=os_)
    else:
        torch.mm(xs, weight.t(), out=os_)
    return out


def linear_split(
    x: torch.Tensor,
    weight: torch.Tensor,
    scratch: torch.Tensor,
    num_rows: int,
    status: torch.Tensor,
) -> Partials:
    """x @ weight.T as float32 split products in ``scratch`` [max_splits, rows, N] (no bias)."""
    splits = min(choose_splits(weight.shape[0], weight.shape[1], num_rows), scratch.shape[0])
    used = kernels.gemm_bf16(x, weight, None, scratch, kernels.GEMM_OUT_F32, num_rows, status, splits=splits)
    return Partials(scratch, used)


def swiglu_linear(
    x: torch.Tensor,
    gate_up_weight: torch.Tensor,
    out: torch.Tensor,
    num_rows: int,
    status: torch.Tensor,
) -> torch.Tensor:
    """out = silu(x @ Wg.T) * (x @ Wu.T) in one kernel (gate and up rows of one matrix)."""
    kernels.gemm_bf16(x, gate_up_weight, None, out, kernels.GEMM_SWIGLU, num_rows, status)
    return out


Pending = Union[torch.Tensor, Partials, None]
