"""Engine and scheduler options, with the reference's names and meanings.

``EngineConfig`` follows engine/config.py:34-75 of the reference and ``SchedulerConfig``
engine/scheduler.py:16-23.  Options of subsystems this engine does not have (prefix caching,
quantization, a quantized cache dtype, a download directory) are left out; ``random_weights``
and ``weights_seed`` are additions.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

_DTYPES = {
    "auto": torch.bfloat16,
    "bfloat16": torch.bfloat16,
    "bf16": torch.bfloat16,
    "float32": torch.float32,
    "fp32": torch.float32,
}


def resolve_dtype(name: str) -> torch.dtype:
    """Map a dtype name to the compute dtype.  ``auto`` is bfloat16: B200 always has it."""
    key = (name or "auto").lower()
    if key not in _DTYPES:
        raise ValueError(f"unknown dtype {name!r}; expected one of {sorted(_DTYPES)}")
    return _DTYPES[key]


@dataclass
class EngineConfig:
    model: str = ""
    dtype: str = "auto"
    device: str = "cuda"

    max_model_len: int = 4096
    max_num_seqs: int = 32
    max_num_batched_tokens: int = 2048
    max_prefill_chunk_size: int = 512

    # Keys per cache page.  64 (the reference's default is 16): a page is then one key tile of
    # the attention kernels and comes in by one tensor-map copy per 64 dims; with smaller
    # pages the copy engines' rate of small copies, not HBM, bounds a decode step.
    block_size: int = 64
    num_gpu_blocks: Optional[int] = None
    gpu_memory_utilization: float = 0.90
    kv_cache_reserve_mb: int = 512

    enable_cuda_graphs: bool = True
    seed: Optional[int] = None

    def torch_dtype(self) -> torch.dtype:
        return resolve_dtype(self.dtype)

    def validate(self) -> None:
        if self.max_num_seqs < 1:
            raise ValueError("max_num_seqs must be at least 1")
        if self.max_prefill_chunk_size < 1:
            raise ValueError("max_prefill_chunk_size must be at least 1")
        if self.max_num_batched_tokens < self.max_prefill_chunk_size:
            raise ValueError("max_num_batched_tokens must be at least max_prefill_chunk_size")
        if self.max_num_batched_tokens < self.max_num_seqs:
            raise ValueError(
                "max_num_batched_tokens must leave room for one token per running sequence"
            )
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            raise ValueError("gpu_memory_utilization must be in (0, 1]")
        if self.block_size <= 0 or (self.block_size & (self.block_size - 1)) != 0:
            raise ValueError("block_size must be a power of two")
        if self.num_gpu_blocks is not None and self.num_gpu_blocks < 2:
            raise ValueError("num_gpu_blocks must be at least 2 (block 0 is reserved)")
        resolve_dtype(self.dtype)


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 32
    max_num_batched_tokens: int = 2048
    max_prefill_chunk_size: int = 512
    max_model_len: int = 4096
    # Fraction of every pool kept free when a new request is admitted (at least one block).
    watermark: float = 0.01
