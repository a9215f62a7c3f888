"""A generation request and its life cycle.

Field names and meanings follow engine/request.py:14-179 of the reference: ``all_token_ids``
is prompt plus generated tokens, ``num_computed_tokens`` counts the tokens whose keys and values
are in the cache, a request *is decoding* when at most one token is not yet computed, and
prefill and decode are the same operation at different chunk sizes.
"""
from __future__ import annotations

import time
from enum import Enum
from typing import Callable, FrozenSet, List, Optional

from ..cache.manager import SequenceCache
from ..sampling.params import SamplingParams


class RequestStatus(Enum):
    WAITING = "waiting"
    RUNNING_PREFILL = "running_prefill"
    RUNNING_DECODE = "running_decode"
    PREEMPTED = "preempted"
    FINISHED = "finished"
    ABORTED = "aborted"


class FinishReason(str, Enum):
    STOP = "stop"
    LENGTH = "length"
    ABORT = "abort"


class Request:
    def __init__(
        self,
        request_id: str,
        prompt_token_ids: List[int],
        sampling_params: Optional[SamplingParams] = None,
        arrival_time: Optional[float] = None,
    ) -> None:
        if not prompt_token_ids:
            raise ValueError("prompt_token_ids must contain at least one token")
        self.request_id = request_id
        self.prompt_token_ids = list(prompt_token_ids)
        self.num_prompt_tokens = len(self.prompt_token_ids)
        self.sampling_params = sampling_params or SamplingParams()
        self.arrival_time = time.time() if arrival_time is None else arrival_time

        self.status = RequestStatus.WAITING
        self.output_token_ids: List[int] = []
        self.all_token_ids: List[int] = list(self.prompt_token_ids)

        # Set by the scheduler when the request is first queued.
        self.cache: Optional[SequenceCache] = None
        self.current_chunk_size = 0

        self.finished = False
        self.finish_reason: Optional[FinishReason] = None
        self.num_preemptions = 0
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None
        self._listeners: List[Callable[["Request", str, Optional[int]], None]] = []

    # ------------------------------------------------------------------ views of the cache state
    @property
    def num_computed_tokens(self) -> int:
        return 0 if self.cache is None else self.cache.num_computed

    @property
    def block_table(self) -> List[int]:
        """Block table of the first cache group."""
        return [] if self.cache is None or not self.cache.tables else self.cache.tables[0]

    @property
    def seq_index(self) -> Optional[int]:
        return None if self.cache is None else self.cache.slot

    # ------------------------------------------------------------------ counts
    @property
    def num_tokens(self) -> int:
        return len(self.all_token_ids)

    @property
    def num_output_tokens(self) -> int:
        return len(self.output_token_ids)

    @property
    def num_uncomputed_tokens(self) -> int:
        return max(0, len(self.all_token_ids) - self.num_computed_tokens)

    @property
    def is_decoding(self) -> bool:
        return self.num_uncomputed_tokens <= 1

    @property
    def max_tokens(self) -> int:
        return self.sampling_params.max_tokens

    def tokens_for_chunk(self, chunk_size: int) -> List[int]:
        start = self.num_computed_tokens
        return self.all_token_ids[start : start + chunk_size]

    # ------------------------------------------------------------------ transitions
    def append_token(self, token_id: int) -> None:
        self.output_token_ids.append(token_id)
        self.all_token_ids.append(token_id)
        if self.first_token_time is None:
            self.first_token_time = time.time()
        self._emit("token", token_id)

    def refresh_status(self) -> None:
        if self.finished:
            return
        self.status = (
            RequestStatus.RUNNING_DECODE if self.is_decoding else RequestStatus.RUNNING_PREFILL
        )

    def should_stop(self, token_id: int, eos_token_ids: FrozenSet[int]) -> Optional[FinishReason]:
        params = self.sampling_params
        if not params.ignore_eos and (
            token_id in eos_token_ids or token_id in params.stop_token_ids
        ):
            return FinishReason.STOP
        if len(self.output_token_ids) >= params.max_tokens:
            return FinishReason.LENGTH
        return None

    def finish(self, reason: FinishReason) -> None:
        if self.finished:
            return
        self.finished = True
        self.finish_reason = reason
        self.finish_time = time.time()
        self.status = (
            RequestStatus.ABORTED if reason is FinishReason.ABORT else RequestStatus.FINISHED
        )
        self._emit("finish", None)

    # ------------------------------------------------------------------ listeners
    def add_listener(self, listener: Callable[["Request", str, Optional[int]], None]) -> None:
        """``listener(request, kind, token_id)`` with kind "token" or "finish"."""
        self._listeners.append(listener)

    def _emit(self, kind: str, token_id: Optional[int]) -> None:
        for listener in self._listeners:
            try:
                listener(self, kind, token_id)
            except Exception:  # a listener must not break the engine loop
                import logging

                logging.getLogger(__name__).exception(
                    "request %s: listener raised", self.request_id
                )

    @property
    def time_to_first_token(self) -> Optional[float]:
        if self.first_token_time is None:
            return None
        return self.first_token_time - self.arrival_time

    def __repr__(self) -> str:
        return (
            f"Request(id={self.request_id}, status={self.status.name}, "
            f"prompt={self.num_prompt_tokens}, computed={self.num_computed_tokens}, "
            f"output={len(self.output_token_ids)})"
        )
