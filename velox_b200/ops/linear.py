"""Matrix products of the model: ``y = x @ W.T + b`` with W stored [out, in].

float32: this package's own FP32-pipe kernel, always (no TF32, no tensor cores): it is the
true 32-bit path and sums every output element in a fixed order.

bfloat16: the tcgen05/TMA kernel of ``csrc/gemm_bf16.cu`` when the step has few tokens (decode
and short portions: the weight fills the 128-row side of the tensor-core tile and is streamed
once; projections with few output tiles are split along K over a thread-block cluster), a
library GEMM (cuBLAS through torch) for long portions and for inner sizes the TMA tiles cannot
take.  The reference engine uses a library GEMM for every projection (``nn.Linear``,
src/self_attention.py:32-33, src/mlp.py:9-10, src/transformer.py:60 of that project).
"""
from __future__ import annotations

import os
from typing import Optional

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


def use_tensor_core_kernel(x, weight: torch.Tensor, num_rows: int) -> bool:
    if _is_pending_norm(x):
        x = x.out
    return (
        weight.dtype == torch.bfloat16
        and num_rows <= SMALL_STEP_TOKENS
        and kernels.gemm_bf16_supported(x, weight)
    )


def _is_pending_norm(x) -> bool:
    return not isinstance(x, torch.Tensor) and hasattr(x, "materialize")


def _fuses_norm(x, weight: torch.Tensor, num_rows: int, status) -> bool:
    """``x`` is a norm that has not run and this projection can make it on the fly."""
    return (
        _is_pending_norm(x)
        and status is not None
        and num_rows <= kernels.GEMM_NORMED_MAX_TOKENS
        and x.resid.dtype == torch.float32
        and x.resid.stride(0) % 4 == 0
        and use_tensor_core_kernel(x, weight, num_rows)
    )


def choose_splits(out_features: int, in_features: int, num_rows: int = 1, tile: int = 128) -> int:
    """CTAs per output tile (a power of two up to 8) so that tiles x splits fills the GPU, with
    at least two 64-wide blocks of the inner dimension each.  With at most 32 tokens an SM holds
    two CTAs of the kernel, and a grid of up to 1.6 CTAs per SM streams faster than one that
    leaves SMs idle (measured at the 7B and 14B sizes: 40 tiles x 4 = 160 CTAs take 43 us for the
    14B down projection, 40 x 2 = 80 take 49); wider token tiles are one CTA per SM."""
    tiles = max(1, -(-out_features // tile))
    blocks = -(-in_features // 64)
    room = _num_sms() * (8 if num_rows <= 32 else 5) // 5
    splits = 1
    while splits * 2 <= min(8, blocks // 2) and tiles * splits * 2 <= room:
        splits *= 2
    return splits


# VELOX_B200_NO_CHUNKED_SPLITK=1 keeps the sums into the residual stream in a fixed order (the
# cluster form of split K), for bisecting.  VELOX_B200_DETERMINISTIC=1 does that and keeps the
# feed-forward of small steps as two kernels: every sum of the bfloat16 path then has a fixed
# order and a run repeats bit by bit (seeded sampling gives the same tokens again), at the
# price of the two fastest forms of small steps.
DETERMINISTIC = os.environ.get("VELOX_B200_DETERMINISTIC") == "1"
_CHUNKED_SPLITK = os.environ.get("VELOX_B200_NO_CHUNKED_SPLITK") != "1" and not DETERMINISTIC


def choose_chunks(out_features: int, in_features: int, num_rows: int, tile: int = 128) -> int:
    """Ranges of the inner dimension for ``kernels.gemm_bf16_add_chunked``: enough CTAs for two
    per SM with at most 32 tokens and one per SM with more (measured: the down projection of the
    14B sizes at 64 tokens takes 49 us as 40 x 3 CTAs, 67 us as 40 clusters of two), each with
    at least two 64-wide blocks (the output projection of the 1.5B sizes at 64 tokens, alone with
    a cold L2: 9.9 us as 12 x 6 CTAs of four blocks, 8.7 us as 12 x 12 of two)."""
    token_tile = 16 if num_rows <= 16 else 32 if num_rows <= 32 else 64 if num_rows <= 64 else 128 if num_rows <= 128 else 256
    tiles = max(1, -(-out_features // tile)) * max(1, -(-num_rows // token_tile))
    room = _num_sms() * (2 if num_rows <= 32 else 1)
    blocks = -(-in_features // 64)
    return max(1, min(room // tiles, blocks // 2))


def linear(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias_f32: Optional[torch.Tensor],
    out: torch.Tensor,
    num_rows: int,
    bias_lowp: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
    accumulate: bool = False,
    mirror: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """out[:num_rows] = x[:num_rows] @ weight.T (+ bias), in the dtype of ``out``.

    ``accumulate`` (tensor-core kernel only, float32 ``out``): add to ``out`` instead, which is
    how a projection goes straight into the float32 residual stream.  With ``mirror`` (float32
    rows) the sums are written there as well, by the same kernel where it can.

    ``x`` may be a ``parts.base.PendingNorm``: with few tokens the norm is then made inside the
    projection, otherwise it runs first.
    """
    if num_rows == 0:
        return out
    if _is_pending_norm(x):
        if not accumulate and _fuses_norm(x, weight, num_rows, status):
            mode = kernels.GEMM_OUT_F32 if out.dtype == torch.float32 else kernels.GEMM_OUT_BF16
            if kernels.gemm_bf16_normed(x.resid, x.weight, x.eps, weight, bias_f32, out, mode, num_rows, status,
                                        splits=choose_splits(weight.shape[0], weight.shape[1], num_rows)):
                return out
        x = x.materialize()
    if weight.dtype == torch.float32:
        if accumulate:
            raise ValueError("the float32 GEMM does not accumulate")
        kernels.gemm_f32(x, weight, bias_f32, out, num_rows)
        return out
    if weight.dtype != torch.bfloat16:
        raise TypeError(f"linear: weights must be float32 or bfloat16, got {weight.dtype}")
    if status is not None and use_tensor_core_kernel(x, weight, num_rows):
        if accumulate and mirror is not None:
            # The kernel writes both where it can (no bias, K split over a cluster); else the
            # sums are copied, so that a caller who passes a mirror always finds it written.
            splits = choose_splits(weight.shape[0], weight.shape[1], num_rows)
            if bias_f32 is not None or not kernels.gemm_bf16_add_mirrored(x, weight, out, mirror, num_rows, status,
                                                                         splits):
                kernels.gemm_bf16(x, weight, bias_f32, out, kernels.GEMM_ADD_F32, num_rows, status, splits=splits)
                mirror[:num_rows].copy_(out[:num_rows])
            return out
        if accumulate:
            chunks = choose_chunks(weight.shape[0], weight.shape[1], num_rows) if _CHUNKED_SPLITK else 1
            if chunks > 1 and bias_f32 is None:
                kernels.gemm_bf16_add_chunked(x, weight, out, num_rows, status, chunks)
                return out
            mode = kernels.GEMM_ADD_F32
        else:
            mode = kernels.GEMM_OUT_F32 if out.dtype == torch.float32 else kernels.GEMM_OUT_BF16
        kernels.gemm_bf16(x, weight, bias_f32, out, mode, num_rows, status,
                          splits=choose_splits(weight.shape[0], weight.shape[1], num_rows))
        return out
    if accumulate:
        raise ValueError("only the tensor-core kernel accumulates into its output")
    if out.dtype != torch.bfloat16:
        raise TypeError("the library GEMM path writes bfloat16")
    xs, os_ = x[:num_rows], out[:num_rows]
    if bias_f32 is not None:
        if bias_lowp is None:
            raise ValueError("the bfloat16 library GEMM needs the bias in bfloat16 too")
        torch.addmm(bias_lowp, xs, _transposed(weight), out=os_)
    else:
        torch.mm(xs, _transposed(weight), out=os_)
    kernels.note_library_launch("library_gemm")
    return out


def _transposed(weight: torch.Tensor) -> torch.Tensor:
    """The transposed view of a weight, made once and kept on the weight itself."""
    view = getattr(weight, "_vx_transposed", None)
    if view is None:
        view = weight.t()
        weight._vx_transposed = view
    return view


def swiglu_linear(
    x: torch.Tensor,
    gate_up_weight: torch.Tensor,
    out: torch.Tensor,
    num_rows: int,
    status: torch.Tensor,
) -> torch.Tensor:
    """out = silu(x @ Wg.T) * (x @ Wu.T) in one kernel (gate and up rows of one matrix)."""
    if _is_pending_norm(x):
        if _fuses_norm(x, gate_up_weight, num_rows, status):
            if kernels.gemm_bf16_normed(x.resid, x.weight, x.eps, gate_up_weight, None, out,
                                        kernels.GEMM_SWIGLU, num_rows, status):
                return out
        x = x.materialize()
    kernels.gemm_bf16(x, gate_up_weight, None, out, kernels.GEMM_SWIGLU, num_rows, status)
    return out


def qkv_rope_linear(
    x,
    weight: torch.Tensor,
    bias_f32: Optional[torch.Tensor],
    out: torch.Tensor,
    num_rows: int,
    status: Optional[torch.Tensor],
    positions: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    slots: torch.Tensor,
    k_cache: Optional[torch.Tensor],
    v_cache: Optional[torch.Tensor],
    num_heads: int,
    num_kv_heads: int,
) -> bool:
    """The QKV projection with the rotation of q and k and the write of k and v into the cache
    in the same kernel (few tokens, heads of 128 dims, a projection that is split along K).
    ``x`` is a tensor or a ``PendingNorm``.  False: nothing was done; the caller projects with
    ``linear`` and rotates with the position part."""
    if status is None or num_rows == 0 or num_rows > kernels.GEMM_NORMED_MAX_TOKENS:
        return False
    if not use_tensor_core_kernel(x, weight, num_rows):
        return False
    splits = choose_splits(weight.shape[0], weight.shape[1], num_rows)
    if splits < 2:
        return False
    if _is_pending_norm(x):
        if _fuses_norm(x, weight, num_rows, status) and kernels.gemm_bf16_qkv_rope(
                None, x.resid, x.weight, x.eps, weight, bias_f32, out, num_rows, positions, cos, sin, slots,
                k_cache, v_cache, num_heads, num_kv_heads, status, splits):
            return True
        x = x.materialize()
    return kernels.gemm_bf16_qkv_rope(x, None, None, 0.0, weight, bias_f32, out, num_rows, positions, cos, sin,
                                      slots, k_cache, v_cache, num_heads, num_kv_heads, status, splits)
