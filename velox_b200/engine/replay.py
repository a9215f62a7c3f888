"""Trace replay: given token ids go through the engine's own step function, logits come back.

A trace is a sequence of steps; a step names, for some requests, their next tokens and the
places among them whose logits are wanted, and the requests that end after it.  Replay samples
nothing and decides nothing: the trace dictates how prompts are cut and what shares a batch.
It drives the same model, cache manager, block tables and kernels as generation does.  The
reference has no such program; its tests reach below ``Engine.step`` by hand for the same
purpose (tests/test_engine_e2e.py:107-124 of that project).
"""
from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import numpy as np
import torch

from ..cache.manager import CacheManager, SequenceCache
from ..config.engine_config import resolve_dtype
from .engine import load_model
from .runner import ModelRunner, StepChunk


class TraceReplayer:
    def __init__(
        self,
        model_dir: str,
        dtype: str,
        max_tokens: int,
        block_size: int = 16,
        max_live: int = 8,
        device: str = "cuda:0",
        plan_overrides: Optional[dict] = None,
        enable_graphs: bool = True,
    ) -> None:
        if block_size < 1 or 64 % block_size != 0:
            raise ValueError("block_size must divide 64")
        self.device = torch.device(device)
        # Every request's token count is rounded up to a multiple of 64 when the pool is sized.
        capacity = -(-max_tokens // 64) * 64
        _, _, self.model = load_model(model_dir, resolve_dtype(dtype), self.device, max_position=capacity)
        self.cache = CacheManager(
            self.model.cache_groups,
            num_pages=capacity // block_size + 1,  # page 0 is reserved
            page_size=block_size,
            max_model_len=capacity,
            max_num_seqs=max_live,
        )
        self.runner = ModelRunner(
            self.model, self.cache, max_num_seqs=max_live, max_num_batched_tokens=capacity,
            plan_overrides=plan_overrides, enable_graphs=enable_graphs,
        )
        self.max_live = max_live
        self.max_tokens = max_tokens
        self.live: Dict[str, SequenceCache] = {}

    def run_step(self, record: Mapping[str, Any]) -> Optional[np.ndarray]:
        """Run one step of a trace; returns float32 logits [wanted, vocab] or None."""
        step = record.get("step")
        chunks = []
        for entry in record.get("entries", []):
            name = str(entry["id"])
            tokens = [int(t) for t in entry["tokens"]]
            if not tokens:
                continue
            seq = self.live.get(name)
            if seq is None:
                seq = self.cache.new_sequence(name)
                if not self.cache.acquire_slot(seq):
                    raise RuntimeError(f"step {step}: more than {self.max_live} live requests")
                self.live[name] = seq
            if not self.cache.append_slots(seq, len(tokens)):
                raise RuntimeError(
                    f"step {step}: no pages left for request {name!r} "
                    f"({seq.num_computed} + {len(tokens)} tokens; max_tokens {self.max_tokens})"
                )
            chunks.append(StepChunk(seq, tokens, tuple(int(w) for w in entry.get("want", []))))
        logits = self.runner.step(chunks) if chunks else None
        for chunk in chunks:
            self.cache.advance(chunk.seq, len(chunk.tokens))
        result = None
        if logits is not None:
            result = np.ascontiguousarray(logits.to("cpu").numpy().astype("<f4", copy=False))
        else:
            torch.cuda.synchronize(self.device)
        self.runner.check_status()
        for name in record.get("end", []):
            seq = self.live.pop(str(name), None)
            if seq is not None:
                self.cache.free(seq)
                self.cache.release_slot(seq)
        return result
