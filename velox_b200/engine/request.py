"""A generation request: its tokens, where it stands, and who wants to hear about it.

The public names are the ones a user of the reference engine knows (engine/request.py of that
project: ``request_id``, ``prompt_token_ids``, ``output_token_ids``, ``all_token_ids``,
``num_computed_tokens``, ``finish_reason`` ...), because requests are part of the Python entry
point.  How they are kept is this engine's own: one token list with the prompt's length as a
mark, the cache bookkeeping in the request's ``SequenceCache`` (``cache``), and a table that
says which status follows from which facts.
"""
from __future__ import annotations

import logging
import time
from enum import Enum
from typing import Callable, FrozenSet, List, Optional, Sequence

from ..cache.manager import SequenceCache
from ..sampling.params import SamplingParams

_log = logging.getLogger(__name__)

Listener = Callable[["Request", str, Optional[int]], None]


class RequestStatus(Enum):
    WAITING = "waiting"
    RUNNING_PREFILL = "running_prefill"
    RUNNING_DECODE = "running_decode"
    PREEMPTED = "preempted"
    FINISHED = "finished"
    ABORTED = "aborted"


class FinishReason(str, Enum):
    STOP = "stop"      # an end-of-sequence or stop token was sampled
    LENGTH = "length"  # max_tokens reached
    ABORT = "abort"    # taken out by the caller


# What a finished request's status is, by the reason it ended for.
_STATUS_AFTER = {
    FinishReason.STOP: RequestStatus.FINISHED,
    FinishReason.LENGTH: RequestStatus.FINISHED,
    FinishReason.ABORT: RequestStatus.ABORTED,
}


class Request:
    """One prompt and what has been generated for it so far.

    A request is *decoding* when at most one of its tokens is not in the cache yet: prefill and
    decode are the same operation on portions of different length, and a preempted request
    simply has all of its tokens (prompt and generated) uncomputed again.
    """

    def __init__(
        self,
        request_id: str,
        prompt_token_ids: Sequence[int],
        sampling_params: Optional[SamplingParams] = None,
        arrival_time: Optional[float] = None,
    ) -> None:
        tokens = [int(t) for t in prompt_token_ids]
        if len(tokens) == 0:
            raise ValueError(f"request {request_id!r}: an empty prompt cannot be continued")
        self.request_id = request_id
        self.sampling_params = SamplingParams() if sampling_params is None else sampling_params
        self.arrival_time = arrival_time if arrival_time is not None else time.time()
        # prompt first, generated tokens after it
        self._tokens: List[int] = tokens
        self._prompt_len = len(tokens)
        # Given by the scheduler at the first queueing; holds the block tables, the state slot
        # and the count of computed tokens.
        self.cache: Optional[SequenceCache] = None
        # Tokens the scheduler gave this request in the step that is being run.
        self.current_chunk_size = 0
        self.status = RequestStatus.WAITING
        self.finish_reason: Optional[FinishReason] = None
        self.num_preemptions = 0
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None
        self._listeners: List[Listener] = []
        # Generated tokens at the end of the list that are only known on the device so far (the
        # list holds a stand-in for each), and whether the end has been told to the listeners.
        self._pending = 0
        self._finish_told = False

    # ------------------------------------------------------------------ tokens
    @property
    def all_token_ids(self) -> List[int]:
        """Prompt and generated tokens, the list itself (what a recompute prefills)."""
        return self._tokens

    @property
    def prompt_token_ids(self) -> List[int]:
        return self._tokens[: self._prompt_len]

    @property
    def output_token_ids(self) -> List[int]:
        """The generated tokens the host knows (a token still on its way from the device is
        counted by ``num_output_tokens`` but not shown here)."""
        return self._tokens[self._prompt_len : len(self._tokens) - self._pending]

    @property
    def num_prompt_tokens(self) -> int:
        return self._prompt_len

    @property
    def num_output_tokens(self) -> int:
        return len(self._tokens) - self._prompt_len

    @property
    def num_tokens(self) -> int:
        return len(self._tokens)

    @property
    def max_tokens(self) -> int:
        return self.sampling_params.max_tokens

    # ------------------------------------------------------------------ what the cache holds
    @property
    def num_computed_tokens(self) -> int:
        return self.cache.num_computed if self.cache is not None else 0

    @property
    def num_uncomputed_tokens(self) -> int:
        return max(len(self._tokens) - self.num_computed_tokens, 0)

    @property
    def is_decoding(self) -> bool:
        return self.num_uncomputed_tokens <= 1

    @property
    def block_table(self) -> List[int]:
        """Pages of the first cache group (all groups have tables of the same length)."""
        if self.cache is None or not self.cache.tables:
            return []
        return self.cache.tables[0]

    @property
    def seq_index(self) -> Optional[int]:
        """The state slot, while the request runs."""
        return self.cache.slot if self.cache is not None else None

    def tokens_for_chunk(self, chunk_size: int) -> List[int]:
        """The next ``chunk_size`` tokens that are not in the cache yet."""
        first = self.num_computed_tokens
        return self._tokens[first : first + chunk_size]

    # ------------------------------------------------------------------ life cycle
    @property
    def finished(self) -> bool:
        return self.finish_reason is not None

    def refresh_status(self) -> None:
        """A running request is in prefill or in decode by how much of it is uncomputed."""
        if not self.finished:
            self.status = RequestStatus.RUNNING_DECODE if self.is_decoding else RequestStatus.RUNNING_PREFILL

    def append_token(self, token_id: int) -> None:
        self._tokens.append(int(token_id))
        if self.first_token_time is None:
            self.first_token_time = time.time()
        self._tell("token", token_id)

    def append_pending(self, stand_in: int) -> int:
        """A token has been drawn on the device and is not known here yet: ``stand_in`` (a
        negative id that the embedding resolves on the device) takes its place.  Returns the
        place, for ``resolve_pending``.  Nobody is told."""
        self._tokens.append(int(stand_in))
        self._pending += 1
        return len(self._tokens) - 1

    def resolve_pending(self, place: int, token_id: int) -> None:
        """The token at ``place`` has arrived: it replaces its stand-in and is announced."""
        self._tokens[place] = int(token_id)
        self._pending -= 1
        if self.first_token_time is None:
            self.first_token_time = time.time()
        self._tell("token", token_id)

    def drop_pending(self, place: int) -> None:
        """The token at ``place`` is not wanted any more (the request ended before it came)."""
        if place == len(self._tokens) - 1 and self._pending > 0:
            self._tokens.pop()
            self._pending -= 1

    def should_stop(self, token_id: int, eos_token_ids: FrozenSet[int]) -> Optional[FinishReason]:
        """Whether the token just appended ends the request, and why."""
        params = self.sampling_params
        ends_text = token_id in eos_token_ids or token_id in params.stop_token_ids
        if ends_text and not params.ignore_eos:
            return FinishReason.STOP
        return FinishReason.LENGTH if self.num_output_tokens >= params.max_tokens else None

    def finish(self, reason: FinishReason, announce: bool = True) -> None:
        """Ends the request once; a second call changes nothing.  With ``announce=False`` the
        listeners hear of it only at ``announce_finish`` (the engine ends a request that has
        reached its length before the last token has come back from the device)."""
        if self.finished:
            return
        self.finish_reason = reason
        self.status = _STATUS_AFTER[reason]
        self.finish_time = time.time()
        if announce:
            self.announce_finish()

    @property
    def finish_announced(self) -> bool:
        return self._finish_told

    def announce_finish(self, reason: Optional[FinishReason] = None) -> None:
        """Tells the listeners of the end, once.  ``reason`` replaces the recorded one (a last
        token that is a stop token ends the request by STOP, not by LENGTH)."""
        if reason is not None and self.finish_reason is not FinishReason.ABORT:
            self.finish_reason = reason
            self.status = _STATUS_AFTER[reason]
        if not self._finish_told:
            self._finish_told = True
            self._tell("finish", None)

    @property
    def time_to_first_token(self) -> Optional[float]:
        return None if self.first_token_time is None else self.first_token_time - self.arrival_time

    # ------------------------------------------------------------------ listeners
    def add_listener(self, listener: Listener) -> None:
        """``listener(request, "token", token_id)`` after every generated token and
        ``listener(request, "finish", None)`` at the end.  A listener that raises is logged and
        does not stop the engine."""
        self._listeners.append(listener)

    def _tell(self, kind: str, token_id: Optional[int]) -> None:
        for listener in self._listeners:
            try:
                listener(self, kind, token_id)
            except Exception:
                _log.exception("request %s: a listener raised on %r", self.request_id, kind)

    def __repr__(self) -> str:
        return (f"<Request {self.request_id} {self.status.value}: {self._prompt_len} prompt + "
                f"{self.num_output_tokens} generated tokens, {self.num_computed_tokens} in the cache>")
