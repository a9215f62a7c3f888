"""Sampler: one token per row of float32 logits, on the device.

Options and their meaning follow the reference's sampler (engine/sampler.py:131-258 of that
project); the kernels and what differs from its torch formulation are described in
``csrc/sampling.cu``.  A batch whose rows are all greedy is one argmax launch.  A seeded request
draws from a counter-based generator keyed by (seed, index of the output token), so its tokens
do not depend on which other requests share its steps; a request without a seed gets one from
the sampler's own seed and the request id.

Per-request token histories (for the penalties) live in a device array with one row per state
slot, as the reference's ``TokenHistory`` does (engine/sampler.py:97-128).
"""
from __future__ import annotations

import hashlib
import os
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..ops import kernels
from .params import SamplingParams

_COLUMNS = 10  # temperature, top_p, top_k, repetition, presence, frequency, seed lo/hi, draw, slot


def _derive_seed(base: int, request_id: str) -> int:
    digest = hashlib.sha256(f"{base}:{request_id}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little")


class TokenReadback:
    """Sampled tokens from the device to the host without stopping the host: ``begin`` queues
    the copy into pinned memory behind the sampling kernel and returns a ticket, ``end`` waits
    for that copy alone and returns the values.  Two buffers, used in turn: two steps' tokens
    can be on their way at a time."""

    def __init__(self, capacity: int) -> None:
        self._host = [torch.zeros(capacity, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._events = [torch.cuda.Event(), torch.cuda.Event()]
        self._flip = 0

    def begin(self, tokens: torch.Tensor):
        index = self._flip
        self._flip ^= 1
        count = int(tokens.numel())
        self._host[index][:count].copy_(tokens, non_blocking=True)
        self._events[index].record()
        return index, count

    def end(self, ticket) -> List[int]:
        index, count = ticket
        self._events[index].synchronize()
        return self._host[index][:count].tolist()


class Sampler:
    def __init__(
        self,
        device: torch.device,
        vocab_size: int,
        max_num_seqs: int,
        max_model_len: int,
        seed: Optional[int] = None,
    ) -> None:
        self.device = device
        self.vocab_size = vocab_size
        self.max_num_seqs = max_num_seqs
        self.max_model_len = max_model_len
        self.base_seed = int.from_bytes(os.urandom(8), "little") if seed is None else int(seed)
        rows = max_num_seqs
        self._host = [torch.zeros((_COLUMNS + 1, rows), dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._events = [torch.cuda.Event(), torch.cuda.Event()]
        self._used = [False, False]
        self._flip = 0
        self._dev = torch.zeros((_COLUMNS + 1, rows), dtype=torch.int32, device=device)
        # One entry more than rows: the device status word can ride behind the tokens.
        self.tokens = torch.zeros(rows + 1, dtype=torch.int32, device=device)
        self._threshold = torch.zeros(rows, dtype=torch.float32, device=device)
        # Made on first use: most workloads never ask for penalties.
        self._history: Optional[torch.Tensor] = None
        self._counts: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ history for penalties
    def _ensure_history(self) -> torch.Tensor:
        if self._history is None:
            self._history = torch.zeros(
                (self.max_num_seqs + 1, self.max_model_len), dtype=torch.int32, device=self.device
            )
        return self._history

    def start_sequence(self, slot: int, token_ids: Sequence[int], params: SamplingParams) -> None:
        """Called when a request takes a state slot: its tokens so far become its history."""
        if not params.has_penalties:
            return
        history = self._ensure_history()
        length = min(len(token_ids), self.max_model_len)
        row = torch.tensor(list(token_ids[:length]), dtype=torch.int32)
        history[slot, :length].copy_(row)

    # ------------------------------------------------------------------ sampling
    def sample(
        self,
        logits: torch.Tensor,
        params: Sequence[SamplingParams],
        request_ids: Sequence[str],
        draw_indices: Sequence[int],
        slots: Optional[Sequence[int]] = None,
        history_lengths: Optional[Sequence[int]] = None,
        status: Optional[torch.Tensor] = None,
    ) -> torch.Tensor:
        """Returns int32 device tokens [R]; the caller decides when to read them back.

        ``draw_indices[r]`` is the index of the output token being drawn for row r.  ``slots``
        and ``history_lengths`` (tokens of the request so far) are needed for the penalties.
        With ``status`` (the runner's device status word) the result has R + 1 entries, the
        last one being that word as it stood when the tokens were drawn: one read-back brings
        both.
        """
        rows = logits.shape[0]
        if len(params) != rows:
            raise ValueError(f"got {len(params)} sampling params for {rows} rows of logits")
        if rows > self.max_num_seqs:
            raise ValueError(f"{rows} rows exceed the sampler's {self.max_num_seqs}")
        out = self.tokens[: rows + (0 if status is None else 1)]
        any_penalty = any(p.has_penalties for p in params)
        if all(p.is_greedy for p in params) and not any_penalty:
            kernels.sample(logits, rows, None, None, None, None, out, status=status)
            return out

        index = self._flip
        self._flip ^= 1
        if self._used[index]:
            self._events[index].synchronize()
        host = self._host[index].numpy()
        as_float = host.view(np.float32)
        # Rows 6 and 7 together hold the 64-bit seeds, one after the other.
        seeds_host = host[6:8].reshape(-1).view(np.uint64)
        for r, p in enumerate(params):
            as_float[0, r] = p.temperature
            as_float[1, r] = p.top_p
            host[2, r] = p.top_k if 0 < p.top_k < self.vocab_size else 0
            as_float[3, r] = p.repetition_penalty
            as_float[4, r] = p.presence_penalty
            as_float[5, r] = p.frequency_penalty
            seed = p.seed if p.seed is not None else _derive_seed(self.base_seed, request_ids[r])
            seeds_host[r] = seed & ((1 << 64) - 1)
            host[8, r] = draw_indices[r]
            host[9, r] = 0 if slots is None else slots[r]
            host[10, r] = 0 if history_lengths is None or not p.has_penalties else history_lengths[r]
        self._dev.copy_(self._host[index], non_blocking=True)
        self._events[index].record()
        self._used[index] = True

        dev = self._dev
        temperature = dev[0, :rows].view(torch.float32)
        top_p = dev[1, :rows].view(torch.float32)
        top_k = dev[2, :rows]
        seeds = dev[6:8].reshape(-1).view(torch.int64)[:rows]
        draw = dev[8, :rows]

        history = None
        if any_penalty:
            if slots is None or history_lengths is None:
                raise ValueError("penalties need the requests' state slots and history lengths")
            history = self._ensure_history()
            if self._counts is None:
                self._counts = torch.zeros(
                    (self.max_num_seqs, self.vocab_size), dtype=torch.int32, device=self.device
                )
            kernels.apply_penalties(
                logits, rows, history, dev[9, :rows], dev[10, :rows], self._counts,
                dev[3, :rows].view(torch.float32), dev[4, :rows].view(torch.float32),
                dev[5, :rows].view(torch.float32),
            )
        threshold = None
        if any(p.filters_candidates and not p.is_greedy for p in params):
            threshold = self._threshold[:rows]
            kernels.filter_threshold(logits, rows, temperature, top_k, top_p, threshold)
        kernels.sample(
            logits, rows, temperature, seeds, draw, threshold, out,
            history, dev[9, :rows] if history is not None else None,
            dev[10, :rows] if history is not None else None,
            status=status,
        )
        return out
