"""Python entry points of the hand-written CUDA kernels (ctypes over the C launchers).

Every function here takes torch tensors that already live on the GPU, checks what a wrong
call could silently get wrong (dtype, contiguity, sizes), and launches on the current torch
stream.  There is no fallback: without a CUDA device or without a working nvcc build these
functions raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc import build

_c_int = ctypes.c_int
_c_ll = ctypes.c_longlong
_c_f = ctypes.c_float
_ptr = ctypes.c_void_p

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}

_core = None
_attention = {}


class KernelError(RuntimeError):
    pass


def _require_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError(
            "velox_b200 runs on a CUDA device only (sm_100a); no CUDA device is available "
            "and there is no CPU path"
        )


def core():
    global _core
    if _core is None:
        lib = build.load_core()
        lib.vx_embed.argtypes = [_ptr, _c_int, _ptr, _ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _c_int, _ptr]
        lib.vx_add_rmsnorm.argtypes = [
            _ptr, _ptr, _ptr, _c_f, _ptr, _c_int, _ptr, _c_int, _c_int, _c_int, _ptr,
        ]
        lib.vx_rope_cache_write.argtypes = [
            _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
            _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_int, _ptr, _ptr,
        ]
        lib.vx_swiglu.argtypes = [_ptr, _ptr, _c_int, _c_int, _c_int, _ptr]
        lib.vx_gemm_f32.argtypes = [_ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _ptr]
        lib.vx_cast_bf16_to_f32.argtypes = [_ptr, _ptr, _c_ll, _ptr]
        lib.vx_sample.argtypes = [
            _ptr, _c_int, _c_int, _c_ll, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_ll, _ptr, _ptr, _ptr, _ptr, _ptr,
            _ptr,
        ]
        lib.vx_sample_segments.argtypes = [_c_int, _c_int]
        lib.vx_selftest_bounded_wait.argtypes = [_ptr, _c_ll, _ptr, _ptr]
        lib.vx_gemm_bf16_add_mirrored.argtypes = [
            _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_int, _ptr, _ptr,
        ]
        lib.vx_mlp_fused.argtypes = [
            _ptr, _c_ll, _ptr, _c_f, _ptr, _ptr, _ptr, _c_ll, _c_int, _c_int, _c_int, _ptr, _ptr,
        ]
        lib.vx_filter_threshold.argtypes = [
            _ptr, _c_int, _c_int, _c_ll, _ptr, _ptr, _ptr, _ptr, _c_int, _ptr,
        ]
        lib.vx_apply_penalties.argtypes = [
            _ptr, _c_int, _c_int, _c_ll, _ptr, _c_ll, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
        ]
        lib.vx_gemm_bf16.argtypes = [
            _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_int, _ptr, _ptr,
        ]
        lib.vx_gemm_bf16_add_chunked.argtypes = [
            _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_int, _ptr, _ptr,
        ]
        lib.vx_gemm_bf16_normed.argtypes = [
            _ptr, _c_ll, _ptr, _c_f, _ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_int, _ptr, _ptr,
        ]
        lib.vx_gemm_bf16_qkv_rope.argtypes = [
            _ptr, _c_int, _ptr, _c_ll, _ptr, _c_f, _ptr, _ptr, _ptr, _c_int, _c_int, _c_ll, _c_int,
            _ptr, _ptr, _ptr, _c_int, _ptr, _ptr, _ptr, _c_ll, _c_int, _c_int, _ptr, _ptr,
        ]
        _core = lib
    return _core


def attention_lib(head_dim: int):
    lib = _attention.get(head_dim)
    if lib is None:
        lib = build.load_attention(head_dim)
        lib.vx_attention.argtypes = [
            _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr,
            _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_int, _c_f, _c_int, _ptr,
        ]
        lib.vx_attn_has_tc.restype = _c_int
        lib.vx_attn_narrow_ctas_per_sm.restype = _c_int
        lib.vx_attn_max_cluster.restype = _c_int
        lib.vx_attn_narrow_max_active_clusters.restype = _c_int
        lib.vx_attn_narrow_max_active_clusters.argtypes = [_c_int]
        lib.vx_attention_merge.argtypes = [
            _c_int, _ptr, _ptr, _ptr, _c_int, _c_int, _ptr, _ptr, _c_int, _c_int, _c_int, _ptr,
        ]
        lib.vx_attn_head_dim.restype = _c_int
        if lib.vx_attn_head_dim() != head_dim:
            raise KernelError(f"attention library for head size {head_dim} reports another size")
        _attention[head_dim] = lib
    return lib


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """Handle of the current device's current stream (asked for at every launch)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


# Launcher calls made so far (each is at least one kernel of this package).
launch_count = 0

# While this is a list, every launcher call appends (launcher name, a CUDA event recorded right
# after its launch).  With the host running ahead of the device (the caller queues a delay
# first), the time between consecutive events is the device time of each launch, without a
# profiler.  An event between two kernels also keeps the second from starting early, so the
# times are those of kernels that run one after the other.
launch_events: Optional[list] = None


def _check(code: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code} at launch")
    if launch_events is not None:
        event = torch.cuda.Event(enable_timing=True)
        event.record()
        launch_events.append((what, event))


def note_library_launch(what: str) -> None:
    """Called after a library kernel (a cuBLAS product through torch) has been queued, so that a
    timeline of ``launch_events`` has an entry for it too.  It does not count as a launch of
    this package's kernels."""
    if launch_events is not None:
        event = torch.cuda.Event(enable_timing=True)
        event.record()
        launch_events.append((what, event))


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if t.dtype is dtype and t.is_cuda and t.is_contiguous():
        return
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"compute dtype must be float32 or bfloat16, got {dtype}") from None


# ------------------------------------------------------------------------------------------
def selftest_bounded_wait(status: torch.Tensor, limit_cycles: int) -> int:
    """Run one CTA that waits, with a limit of ``limit_cycles`` SM cycles, on a barrier nobody
    arrives at.  Returns 1 when the wait gave up (and set its bit in ``status``), 2 if the
    barrier flipped, 0 if the kernel never reported.  Synchronises."""
    _need(status, torch.int32, "status")
    returned = torch.zeros(1, dtype=torch.int32, device=status.device)
    _check(core().vx_selftest_bounded_wait(_p(status), int(limit_cycles), _p(returned), _stream()),
           "selftest_bounded_wait")
    return int(returned.item())


def embed(table: torch.Tensor, ids: torch.Tensor, resid: torch.Tensor, status: torch.Tensor,
          fed: Optional[torch.Tensor] = None) -> None:
    """resid[t, :] = float32(table[ids[t], :]); ids outside the table set a status bit.

    With ``fed`` (int32 on the device: the tokens the sampler drew in the step before, one per
    row) an id of ``-1 - r`` stands for ``fed[r]`` and is looked up on the device."""
    _need(ids, torch.int32, "ids")
    if fed is not None:
        _need(fed, torch.int32, "fed")
    _need(resid, torch.float32, "resid")
    _need(table, table.dtype, "table")
    vocab, hidden = table.shape
    n = ids.numel()
    if resid.shape[0] < n or resid.shape[1] != hidden:
        raise ValueError(f"resid {tuple(resid.shape)} cannot hold {n} rows of width {hidden}")
    _check(
        core().vx_embed(_p(table), _code(table.dtype), _p(ids), _p(resid), n, hidden, vocab,
                        _p(status), _p(fed), 0 if fed is None else fed.numel(), _stream()),
        "embed",
    )


def add_rmsnorm(
    resid: torch.Tensor,
    delta: Optional[torch.Tensor],
    weight: torch.Tensor,
    eps: float,
    out: torch.Tensor,
    num_rows: int,
    rows: Optional[torch.Tensor] = None,
    write_resid: bool = True,
) -> None:
    """v = resid + delta; resid = v (if write_resid); out = rmsnorm(v) * weight, float32 inside.

    ``delta`` is a pending product in the compute dtype, or None.  With ``rows`` (int32
    indices), output row o is computed from input row rows[o].
    """
    _need(resid, torch.float32, "resid")
    _need(weight, torch.float32, "weight")
    _need(out, out.dtype, "out")
    hidden = resid.shape[1]
    if weight.numel() != hidden or out.shape[1] != hidden:
        raise ValueError("norm weight / output width does not match the residual width")
    if delta is not None:
        _need(delta, out.dtype, "delta")
        if delta.shape[1] != hidden:
            raise ValueError("delta width does not match the residual width")
    if rows is not None:
        _need(rows, torch.int32, "rows")
        if rows.numel() < num_rows:
            raise ValueError(f"{num_rows} rows asked for, the index array names {rows.numel()}")
    elif resid.shape[0] < num_rows or (delta is not None and delta.shape[0] < num_rows):
        raise ValueError(f"{num_rows} rows asked for, the input has {resid.shape[0]}")
    if out.shape[0] < num_rows:
        raise ValueError(f"{num_rows} rows asked for, the output holds {out.shape[0]}")
    _check(
        core().vx_add_rmsnorm(_p(resid), _p(delta), _p(weight), float(eps), _p(out),
                              _code(out.dtype), _p(rows), num_rows, hidden,
                              1 if write_resid else 0, _stream()),
        "add_rmsnorm",
    )


def rope_cache_write(
    qkv: torch.Tensor,
    positions: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    slots: torch.Tensor,
    k_cache: Optional[torch.Tensor],
    v_cache: Optional[torch.Tensor],
    num_tokens: int,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    rotary_dim: int,
    status: torch.Tensor,
) -> None:
    """Rotate q in place; rotate k and write k, v to the paged cache at ``slots``.

    ``k_cache``/``v_cache`` None: rotate q only (a layer that reads another layer's cache).
    """
    _need(qkv, qkv.dtype, "qkv")
    _need(positions, torch.int32, "positions")
    _need(slots, torch.int32, "slots")
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise ValueError("qkv width does not match the head counts")
    write = k_cache is not None
    if write:
        _need(k_cache, qkv.dtype, "k_cache")
        _need(v_cache, qkv.dtype, "v_cache")
        num_slots = k_cache.shape[0] * k_cache.shape[1]
    else:
        num_slots = 0
    if rotary_dim > 0:
        _need(cos, torch.float32, "cos")
        _need(sin, torch.float32, "sin")
        max_pos = cos.shape[0]
        if cos.shape[1] != rotary_dim // 2:
            raise ValueError("cos/sin tables do not match the rotary width")
    else:
        max_pos = 0
    _check(
        core().vx_rope_cache_write(_p(qkv), _code(qkv.dtype), _p(positions), _p(cos), _p(sin),
                                   _p(slots), _p(k_cache), _p(v_cache), num_tokens, num_heads,
                                   num_kv_heads, head_dim, rotary_dim, max_pos, num_slots,
                                   1 if write else 0, _p(status), _stream()),
        "rope_cache_write",
    )


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, num_tokens: int) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _need(gate_up, gate_up.dtype, "gate_up")
    _need(out, gate_up.dtype, "out")
    inter = out.shape[1]
    if gate_up.shape[1] != 2 * inter:
        raise ValueError("gate_up must be twice as wide as the output")
    _check(
        core().vx_swiglu(_p(gate_up), _p(out), _code(out.dtype), num_tokens, inter, _stream()),
        "swiglu",
    )


def gemm_f32(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
             num_rows: int) -> None:
    """out[:M] = a[:M] @ w.T + bias on the FP32 pipes (true 32-bit, no tensor cores)."""
    _need(a, torch.float32, "a")
    _need(w, torch.float32, "w")
    _need(out, torch.float32, "out")
    n, k = w.shape
    if a.shape[1] != k or out.shape[1] != n:
        raise ValueError(f"gemm shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != n:
            raise ValueError("bias length does not match the output width")
    _check(core().vx_gemm_f32(_p(a), _p(w), _p(bias), _p(out), num_rows, n, k, _stream()), "gemm_f32")


GEMM_OUT_BF16, GEMM_OUT_F32, GEMM_ADD_F32, GEMM_SWIGLU = 0, 1, 2, 3


def gemm_bf16_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """The tensor-core kernel moves tiles with TMA: rows must be 16-byte multiples."""
    return w.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def gemm_bf16(
    x: torch.Tensor,
    w: torch.Tensor,
    bias: Optional[torch.Tensor],
    out: torch.Tensor,
    mode: int,
    num_rows: int,
    status: torch.Tensor,
    splits: int = 1,
) -> None:
    """out = x[:num_rows] @ w.T on tcgen05 tensor cores (see gemm_bf16.cu for the modes).

    ``splits`` CTAs (1, 2, 4 or 8; rounded down) share each output tile as a thread-block
    cluster and reduce through distributed shared memory; the output is final either way.
    """
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    n, k = w.shape
    if mode == GEMM_SWIGLU:
        if n % 2:
            raise ValueError("a gate/up matrix needs an even number of rows")
        n //= 2
    if x.shape[1] != k:
        raise ValueError(f"gemm shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}")
    want = torch.bfloat16 if mode in (GEMM_OUT_BF16, GEMM_SWIGLU) else torch.float32
    _need(out, want, "out")
    if out.dim() != 2 or out.shape[1] != n:
        raise ValueError(f"output {tuple(out.shape)} does not match width {n}")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    code = core().vx_gemm_bf16(_p(x), _p(w), _p(bias), _p(out), mode, num_rows, x.shape[0], n, k,
                               out.stride(0), splits, _p(status), _stream())
    if code == -1:
        raise KernelError(
            f"gemm_bf16 refuses x {tuple(x.shape)} w {tuple(w.shape)}: the inner size must be a "
            "multiple of 8 and both operands 16-byte aligned"
        )
    _check(code, "gemm_bf16")


def gemm_bf16_add_chunked(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, num_rows: int,
                          status: torch.Tensor, chunks: int) -> None:
    """out[:num_rows] += x[:num_rows] @ w.T (float32 ``out``) with the inner dimension cut into
    ``chunks`` ranges taken by independent CTAs, which add their partial tiles to ``out`` by
    reductions at the L2: any number of CTAs per output tile, no cluster, and an order of
    additions that is not fixed."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    _need(out, torch.float32, "out")
    n, k = w.shape
    if x.shape[1] != k or out.dim() != 2 or out.shape[1] != n:
        raise ValueError(f"gemm shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    code = core().vx_gemm_bf16_add_chunked(_p(x), _p(w), _p(out), num_rows, x.shape[0], n, k, out.stride(0),
                                           int(chunks), _p(status), _stream())
    if code == -1:
        raise KernelError(f"gemm_bf16_add_chunked refuses x {tuple(x.shape)} w {tuple(w.shape)}")
    _check(code, "gemm_bf16_add_chunked")


# Steps of at most this many tokens can have their input norm made inside the projection.
GEMM_NORMED_MAX_TOKENS = 64


def gemm_bf16_normed(
    resid: torch.Tensor,
    norm_weight: torch.Tensor,
    eps: float,
    w: torch.Tensor,
    bias: Optional[torch.Tensor],
    out: torch.Tensor,
    mode: int,
    num_rows: int,
    status: torch.Tensor,
    splits: int = 1,
) -> bool:
    """``gemm_bf16`` on ``rmsnorm(resid[:num_rows]) * norm_weight`` without that tensor ever
    existing: the kernel makes the bf16 tiles from the float32 rows and applies 1 / rms to its
    accumulator.  At most ``GEMM_NORMED_MAX_TOKENS`` rows.  False (and nothing launched) when
    the tiles of a row this long do not fit in shared memory."""
    if resid.dtype != torch.float32 or resid.dim() != 2 or resid.stride(1) != 1:
        raise TypeError("resid must be float32 rows")
    _need(norm_weight, torch.float32, "norm_weight")
    _need(w, torch.bfloat16, "w")
    n, k = w.shape
    if mode == GEMM_SWIGLU:
        if n % 2:
            raise ValueError("a gate/up matrix needs an even number of rows")
        n //= 2
    if resid.dim() != 2 or resid.shape[1] != k or norm_weight.numel() != k:
        raise ValueError(f"gemm shapes do not agree: resid {tuple(resid.shape)}, w {tuple(w.shape)}")
    if num_rows > GEMM_NORMED_MAX_TOKENS:
        raise ValueError(f"gemm_bf16_normed takes at most {GEMM_NORMED_MAX_TOKENS} rows, got {num_rows}")
    want = torch.bfloat16 if mode in (GEMM_OUT_BF16, GEMM_SWIGLU) else torch.float32
    _need(out, want, "out")
    if out.dim() != 2 or out.shape[1] != n:
        raise ValueError(f"output {tuple(out.shape)} does not match width {n}")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    code = core().vx_gemm_bf16_normed(_p(resid), resid.stride(0), _p(norm_weight), float(eps), _p(w), _p(bias),
                                      _p(out), mode, num_rows, n, k, out.stride(0), splits, _p(status), _stream())
    if code == -2:
        return False
    if code == -1:
        raise KernelError(
            f"gemm_bf16_normed refuses resid {tuple(resid.shape)} w {tuple(w.shape)}: the inner size must "
            "be a multiple of 8, the row pitch of resid a multiple of 4 and the operands 16-byte aligned"
        )
    _check(code, "gemm_bf16_normed")
    return True


def gemm_bf16_add_mirrored(
    x: torch.Tensor,
    w: torch.Tensor,
    out: torch.Tensor,
    mirror: torch.Tensor,
    num_rows: int,
    status: torch.Tensor,
    splits: int,
) -> bool:
    """out[:num_rows] += x[:num_rows] @ w.T (float32) with the sums also written to ``mirror``:
    a copy of the rows that stays as it is while a later kernel adds to ``out`` again.  False
    (nothing launched) where the launch would not be split along K."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    _need(out, torch.float32, "out")
    if mirror.dtype != torch.float32 or mirror.dim() != 2 or mirror.stride(1) != 1 or mirror.shape[1] != out.shape[1]:
        raise TypeError("mirror must be float32 rows of the width of out")
    n, k = w.shape
    if x.shape[1] != k or out.shape[1] != n:
        raise ValueError(f"gemm shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    code = core().vx_gemm_bf16_add_mirrored(_p(x), _p(w), _p(out), _p(mirror), num_rows, x.shape[0], n, k,
                                            out.stride(0), mirror.stride(0), splits, _p(status), _stream())
    if code in (-1, -4):
        return False
    _check(code, "gemm_bf16_add_mirrored")
    return True


# Steps of at most this many tokens can run the gated feed-forward as one kernel.
MLP_FUSED_MAX_TOKENS = 32


def mlp_fused(
    resid_in: torch.Tensor,
    norm_weight: torch.Tensor,
    eps: float,
    w_gate_up: torch.Tensor,
    w_down: torch.Tensor,
    resid_out: torch.Tensor,
    num_rows: int,
    status: torch.Tensor,
) -> bool:
    """resid_out[:num_rows] += w_down @ (silu(gate) * up) of rmsnorm(resid_in[:num_rows]) *
    norm_weight, in one kernel (see ``mlp_fused_kernel`` in gemm_bf16.cu): the norm is made on
    the spot, the activations stay on the SM, and the CTAs' shares of the sum over the inner
    width meet in ``resid_out`` by float32 reductions at the L2, whose order is not fixed.
    ``resid_in`` and ``resid_out`` are float32 rows and must not overlap (other CTAs add to
    the output while a CTA still reads its input).  False (nothing launched) when the sizes
    do not fit: more than ``MLP_FUSED_MAX_TOKENS`` rows, a width that is no multiple of 128 or
    too long for shared or tensor memory, an inner width that is no multiple of 64."""
    for name, t in (("resid_in", resid_in), ("resid_out", resid_out)):
        if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1 or not t.is_cuda:
            raise TypeError(f"{name} must be float32 rows on the device")
    _need(norm_weight, torch.float32, "norm_weight")
    _need(w_gate_up, torch.bfloat16, "w_gate_up")
    _need(w_down, torch.bfloat16, "w_down")
    width = resid_in.shape[1]
    inner = w_down.shape[1]
    if w_gate_up.shape != (2 * inner, width) or w_down.shape[0] != width or resid_out.shape[1] != width:
        raise ValueError(
            f"mlp_fused shapes do not agree: rows of {width}, gate|up {tuple(w_gate_up.shape)}, down {tuple(w_down.shape)}")
    if norm_weight.numel() != width:
        raise ValueError("mlp_fused: the norm weight has another width than the rows")
    if num_rows > MLP_FUSED_MAX_TOKENS or width % 128 or inner % 64 or resid_in.stride(0) % 4:
        return False
    if resid_in.data_ptr() == resid_out.data_ptr():
        raise ValueError("mlp_fused: resid_in and resid_out must be different buffers")
    code = core().vx_mlp_fused(_p(resid_in), resid_in.stride(0), _p(norm_weight), float(eps), _p(w_gate_up),
                               _p(w_down), _p(resid_out), resid_out.stride(0), num_rows, width, inner,
                               _p(status), _stream())
    if code in (-1, -2):
        return False
    _check(code, "mlp_fused")
    return True


def gemm_bf16_qkv_rope(
    x: Optional[torch.Tensor],
    resid: Optional[torch.Tensor],
    norm_weight: Optional[torch.Tensor],
    eps: float,
    w: torch.Tensor,
    bias: Optional[torch.Tensor],
    out: torch.Tensor,
    num_rows: int,
    positions: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    slots: torch.Tensor,
    k_cache: Optional[torch.Tensor],
    v_cache: Optional[torch.Tensor],
    num_heads: int,
    num_kv_heads: int,
    status: torch.Tensor,
    splits: int,
) -> bool:
    """The QKV projection of heads of 128 dims with rotate-half RoPE and the cache write in its
    epilogue: rotated queries go to ``out`` [rows, (heads + 2 kv_heads) * 128] (its key and
    value columns are left as they are), rotated keys and the values into the paged caches at
    ``slots`` (None caches: no write).  The input is ``x`` (bfloat16) or, when ``resid`` is
    given, ``rmsnorm(resid) * norm_weight``.  False, with nothing launched, for shapes the
    kernel does not take (then project and rotate separately)."""
    _need(w, torch.bfloat16, "w")
    _need(out, torch.bfloat16, "out")
    _need(positions, torch.int32, "positions")
    _need(slots, torch.int32, "slots")
    _need(cos, torch.float32, "cos")
    _need(sin, torch.float32, "sin")
    n, k = w.shape
    if n != (num_heads + 2 * num_kv_heads) * 128 or out.shape[1] != n or cos.shape[1] != 64:
        return False
    if num_rows > GEMM_NORMED_MAX_TOKENS:
        return False
    if resid is not None:
        if resid.dtype != torch.float32 or resid.stride(1) != 1 or resid.shape[1] != k:
            raise TypeError("resid must be float32 rows as wide as the weight")
        _need(norm_weight, torch.float32, "norm_weight")
    else:
        _need(x, torch.bfloat16, "x")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    write = k_cache is not None
    if write:
        _need(k_cache, torch.bfloat16, "k_cache")
        _need(v_cache, torch.bfloat16, "v_cache")
        if k_cache.shape[2] != num_kv_heads or k_cache.shape[3] != 128:
            return False
    num_slots = k_cache.shape[0] * k_cache.shape[1] if write else 0
    code = core().vx_gemm_bf16_qkv_rope(
        _p(x), 0 if x is None else x.shape[0], _p(resid), 0 if resid is None else resid.stride(0),
        _p(norm_weight), float(eps), _p(w), _p(bias), _p(out), num_rows, k, out.stride(0), splits,
        _p(positions), _p(cos), _p(sin), cos.shape[0], _p(slots), _p(k_cache), _p(v_cache), num_slots,
        num_heads, num_kv_heads, _p(status), _stream())
    if code in (-1, -2):
        return False
    _check(code, "gemm_bf16_qkv_rope")
    return True


def cast_bf16_to_f32(src: torch.Tensor, out: torch.Tensor, count: int) -> None:
    _need(src, torch.bfloat16, "src")
    _need(out, torch.float32, "out")
    _check(core().vx_cast_bf16_to_f32(_p(src), _p(out), count, _stream()), "cast")


# ------------------------------------------------------------------------------------------
ATTN_F32, ATTN_BF16_WIDE, ATTN_BF16_NARROW, ATTN_BF16_TC = 0, 1, 2, 3


def tile_rows(kind: int) -> int:
    return {ATTN_BF16_WIDE: 64, ATTN_BF16_TC: 128}.get(kind, 16)


def attention(
    kind: int,
    q: torch.Tensor,
    out: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_tables: torch.Tensor,
    q_start: torch.Tensor,
    q_len: torch.Tensor,
    kv_len: torch.Tensor,
    items: torch.Tensor,
    num_items: int,
    partial_o: Optional[torch.Tensor],
    partial_lse: Optional[torch.Tensor],
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    window: Optional[int],
    softmax_scale: float,
    merge_items: Optional[torch.Tensor] = None,
    split_counters: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
    cluster: int = 1,
    layout_checked: bool = False,
) -> None:
    """Run ``num_items`` work items (see attention.cu for their layout) of one kernel family.

    ``layout_checked``: the caller has passed these same index and scratch tensors before (the
    step's layout is shared by all layers); only q, out and the caches are checked again.

    With ``merge_items`` and ``split_counters`` (int32, zero, one per merge item and KV head)
    the bfloat16 families merge split key ranges themselves: the last split to finish does it.
    ``cluster`` (1, 2, 4 or 8; narrow bfloat16 family) CTAs share every item as a thread-block
    cluster: each takes a run of the item's key tiles and they merge through distributed shared
    memory.  For the tensor-memory family 2 asks for two CTAs on an SM whatever the grid's size
    (the caller knows that the items' key ranges are long).
    """
    want = torch.float32 if kind == ATTN_F32 else torch.bfloat16
    _need(q, want, "q")
    _need(out, want, "out")
    _need(k_cache, want, "k_cache")
    _need(v_cache, want, "v_cache")
    if k_cache.shape[2] != num_kv_heads or k_cache.shape[3] != head_dim:
        raise ValueError(f"cache shape {tuple(k_cache.shape)} does not match {num_kv_heads} x {head_dim}")
    if not layout_checked:
        for name, t in (("block_tables", block_tables), ("q_start", q_start), ("q_len", q_len),
                        ("kv_len", kv_len), ("items", items)):
            _need(t, torch.int32, name)
        if num_heads % num_kv_heads != 0:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if partial_o is not None:
            _need(partial_o, torch.float32, "partial_o")
            _need(partial_lse, torch.float32, "partial_lse")
        if split_counters is not None:
            _need(split_counters, torch.int32, "split_counters")
            _need(merge_items, torch.int32, "merge_items")
    lib = attention_lib(head_dim)
    _check(
        lib.vx_attention(kind, _p(q), _p(out), _p(k_cache), _p(v_cache), _p(block_tables),
                         _p(q_start), _p(q_len), _p(kv_len), _p(items), num_items,
                         _p(status if status is not None else _attention_status()),
                         _p(partial_o), _p(partial_lse), _p(merge_items), _p(split_counters),
                         q.shape[1], out.shape[1],
                         block_tables.shape[1], num_kv_heads, num_heads // num_kv_heads,
                         k_cache.shape[1], k_cache.shape[0], int(window or 0), float(softmax_scale),
                         int(cluster), _stream()),
        "attention",
    )


def attention_has_tc(head_dim: int) -> bool:
    """Whether prompt portions of this head size run on the tensor-memory (tcgen05) family."""
    return bool(attention_lib(head_dim).vx_attn_has_tc())


def narrow_attention_slots(head_dim: int) -> int:
    """Work items of the narrow bfloat16 family that one SM holds at a time."""
    return int(attention_lib(head_dim).vx_attn_narrow_ctas_per_sm())


def max_attention_cluster(head_dim: int) -> int:
    return int(attention_lib(head_dim).vx_attn_max_cluster())


def attention_cluster_limits(head_dim: int) -> tuple:
    """((cluster size, clusters of that size the device holds at a time), ...), largest first."""
    _require_cuda()
    lib = attention_lib(head_dim)
    limits = []
    size = max_attention_cluster(head_dim)
    while size >= 2:
        count = int(lib.vx_attn_narrow_max_active_clusters(size))
        if count < 0:
            raise KernelError(f"cluster occupancy query for size {size}: CUDA error {-count}")
        limits.append((size, count))
        size //= 2
    return tuple(limits)


_default_status = None


def _attention_status() -> torch.Tensor:
    """A status word for callers that pass none (bounded waits need somewhere to report)."""
    global _default_status
    if _default_status is None:
        _default_status = torch.zeros(4, dtype=torch.int32, device="cuda")
    return _default_status


def attention_merge(
    out: torch.Tensor,
    q_start: torch.Tensor,
    merge_items: torch.Tensor,
    num_items: int,
    partial_o: torch.Tensor,
    partial_lse: torch.Tensor,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    max_rows: int = 64,
) -> None:
    """Combine the splits of the merge items; ``max_rows`` bounds the rows of any item."""
    _need(merge_items, torch.int32, "merge_items")
    lib = attention_lib(head_dim)
    _check(
        lib.vx_attention_merge(_code(out.dtype), _p(out), _p(q_start), _p(merge_items), num_items,
                               max_rows, _p(partial_o), _p(partial_lse), out.shape[1], num_kv_heads,
                               num_heads // num_kv_heads, _stream()),
        "attention_merge",
    )


# ------------------------------------------------------------------------------------------
# Scratch of the sampling kernel per device: the segments' best entries and the rows' arrival
# counters (zero between launches; the kernel puts them back).
_sample_scratch: dict = {}


def _sample_scratch_for(device: torch.device, num_rows: int, vocab: int):
    segments = core().vx_sample_segments(num_rows, vocab)
    if segments <= 1:
        return None, None
    key = (device.type, device.index)
    held = _sample_scratch.get(key)
    if held is None or held[0].shape[0] < num_rows * segments or held[1].shape[0] < num_rows:
        rows = max(num_rows, 64)
        held = (
            torch.zeros((rows * 64, 2), dtype=torch.int32, device=device),
            torch.zeros(rows, dtype=torch.int32, device=device),
        )
        _sample_scratch[key] = held
    return held


def sample(
    logits: torch.Tensor,
    num_rows: int,
    temperature: Optional[torch.Tensor],
    seeds: Optional[torch.Tensor],
    draw_index: Optional[torch.Tensor],
    threshold: Optional[torch.Tensor],
    out: torch.Tensor,
    history: Optional[torch.Tensor] = None,
    history_slots: Optional[torch.Tensor] = None,
    history_lengths: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
) -> None:
    """One token per row: argmax where temperature is 0 (or None), else the exponential race.

    With ``history`` (int32 [slots, width]) the token of row r is also stored at
    ``history[history_slots[r], history_lengths[r]]``.  With ``status`` (the device status
    word) its first entry is copied to ``out[num_rows]``, so ``out`` needs one entry more."""
    _need(logits, torch.float32, "logits")
    _need(out, torch.int32, "out")
    if out.numel() < num_rows + (0 if status is None else 1):
        raise ValueError("out is too short for the rows (and the status word)")
    if temperature is not None:
        _need(temperature, torch.float32, "temperature")
        _need(seeds, torch.int64, "seeds")
        _need(draw_index, torch.int32, "draw_index")
    partial, counters = _sample_scratch_for(logits.device, num_rows, logits.shape[1])
    _check(
        core().vx_sample(_p(logits), num_rows, logits.shape[1], logits.stride(0), _p(temperature),
                         _p(seeds), _p(draw_index), _p(threshold), _p(out), _p(history),
                         0 if history is None else history.stride(0), _p(history_slots),
                         _p(history_lengths), _p(partial), _p(counters), _p(status), _stream()),
        "sample",
    )


def filter_threshold(
    logits: torch.Tensor,
    num_rows: int,
    temperature: torch.Tensor,
    top_k: torch.Tensor,
    top_p: torch.Tensor,
    threshold: torch.Tensor,
    kind: int = 0,
) -> None:
    """threshold[r]: the smallest scaled logit that is a top-k / top-p candidate of row r.

    ``kind`` picks the kernel: 0 a cluster of eight CTAs per row where the row fits their
    registers (196,608 entries) and one CTA per row otherwise, 1 always one CTA per row, 2 the
    cluster kernel or an error.  Both give the same threshold bit for bit."""
    _need(logits, torch.float32, "logits")
    _need(temperature, torch.float32, "temperature")
    _need(top_k, torch.int32, "top_k")
    _need(top_p, torch.float32, "top_p")
    _need(threshold, torch.float32, "threshold")
    _check(
        core().vx_filter_threshold(_p(logits), num_rows, logits.shape[1], logits.stride(0),
                                   _p(temperature), _p(top_k), _p(top_p), _p(threshold), kind, _stream()),
        "filter_threshold",
    )


def apply_penalties(
    logits: torch.Tensor,
    num_rows: int,
    history: torch.Tensor,
    slots: torch.Tensor,
    lengths: torch.Tensor,
    counts: torch.Tensor,
    repetition: torch.Tensor,
    presence: torch.Tensor,
    frequency: torch.Tensor,
) -> None:
    _need(logits, torch.float32, "logits")
    _need(history, torch.int32, "history")
    _need(slots, torch.int32, "slots")
    _need(lengths, torch.int32, "lengths")
    _need(counts, torch.int32, "counts")
    _check(
        core().vx_apply_penalties(_p(logits), num_rows, logits.shape[1], logits.stride(0),
                                  _p(history), history.stride(0), _p(slots), _p(lengths),
                                  _p(counts), _p(repetition), _p(presence), _p(frequency),
                                  _stream()),
        "apply_penalties",
    )
