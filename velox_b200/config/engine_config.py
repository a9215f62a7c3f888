"""Options of the engine and of its scheduler.

The option names, their meanings and their defaults are the reference's (engine/config.py and
the scheduler's own options in engine/scheduler.py of that project), since they are what a
user passes to ``Engine.from_pretrained`` and to the command line.  Left out: the options of
subsystems that do not exist here (prefix caching, quantized weights or cache, a download
directory).  ``block_size`` defaults to 64 instead of 16.

Every option is declared once, as a dataclass field whose metadata carries its check; one loop
validates them all, and the relations between options are a second, short list.
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, Callable, Optional, Tuple

import torch

# Compute dtypes by the names accepted for them.  "auto" is bfloat16: a B200 always has it.
_DTYPE_NAMES: Tuple[Tuple[torch.dtype, Tuple[str, ...]], ...] = (
    (torch.bfloat16, ("auto", "bfloat16", "bf16")),
    (torch.float32, ("float32", "fp32")),
)


def resolve_dtype(name: Optional[str]) -> torch.dtype:
    """The compute dtype a name stands for (case does not matter; nothing means "auto")."""
    wanted = "auto" if not name else name.lower()
    for dtype, names in _DTYPE_NAMES:
        if wanted in names:
            return dtype
    known = sorted(n for _, names in _DTYPE_NAMES for n in names)
    raise ValueError(f"unknown dtype {name!r}; expected one of {known}")


def _option(default: Any, check: Optional[Callable[[Any], bool]] = None, must: str = "") -> Any:
    """A dataclass field with a check on its value and the words for the error."""
    return field(default=default, metadata={"check": check, "must": must})


def _power_of_two(value: int) -> bool:
    return value > 0 and value & (value - 1) == 0


@dataclass
class EngineConfig:
    # what to load and how to compute
    model: str = ""
    dtype: str = _option("auto", lambda v: resolve_dtype(v) is not None, "name a compute dtype")
    device: str = "cuda"
    seed: Optional[int] = None

    # the shape of a step
    max_model_len: int = _option(4096, lambda v: v >= 1, "be at least 1")
    max_num_seqs: int = _option(32, lambda v: v >= 1, "be at least 1")
    max_num_batched_tokens: int = _option(2048, lambda v: v >= 1, "be at least 1")
    max_prefill_chunk_size: int = _option(512, lambda v: v >= 1, "be at least 1")
    enable_cuda_graphs: bool = True
    # ``Engine.generate`` queues a step on the device before it has read the tokens of the step
    # before (which the new step takes from the sampler's device buffer); False: one step at a
    # time, as ``Engine.step`` always does.
    pipeline_decode: bool = True

    # the cache.  A page of 64 keys is one key tile of the attention kernels and arrives by one
    # tensor-map copy per 64 dims; with smaller pages the copy engines' rate of small copies,
    # not HBM, bounds a decode step.
    block_size: int = _option(64, _power_of_two, "be a power of two")
    num_gpu_blocks: Optional[int] = _option(None, lambda v: v is None or v >= 2,
                                            "be at least 2 (block 0 is reserved)")
    gpu_memory_utilization: float = _option(0.90, lambda v: 0.0 < v <= 1.0, "be in (0, 1]")
    kv_cache_reserve_mb: int = _option(512, lambda v: v >= 0, "not be negative")

    def torch_dtype(self) -> torch.dtype:
        return resolve_dtype(self.dtype)

    def validate(self) -> None:
        """ValueError naming the option that cannot be honoured."""
        for option in fields(self):
            check = option.metadata.get("check")
            if check is not None and not check(getattr(self, option.name)):
                raise ValueError(f"{option.name} must {option.metadata['must']}, got {getattr(self, option.name)!r}")
        # A step has to hold a whole prefill portion, and one token of every running request.
        for smaller in ("max_prefill_chunk_size", "max_num_seqs"):
            if self.max_num_batched_tokens < getattr(self, smaller):
                raise ValueError(f"max_num_batched_tokens must be at least {smaller} "
                                 f"({self.max_num_batched_tokens} < {getattr(self, smaller)})")


@dataclass
class SchedulerConfig:
    """What the scheduler needs of the options above, and its own watermark: the fraction of
    every page pool (one page at least) that admitting a new request leaves free."""

    max_num_seqs: int = 32
    max_num_batched_tokens: int = 2048
    max_prefill_chunk_size: int = 512
    max_model_len: int = 4096
    watermark: float = 0.01
