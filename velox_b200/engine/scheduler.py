"""Continuous-batching scheduler: who runs in the next step, and with how many tokens.

The decisions are those of the reference's scheduler (engine/scheduler.py:161-291):

* finished requests are reaped at the start of the next ``schedule()``;
* decoding requests go first, one token each, while the token budget lasts;
* running prefills continue with their next portion, ``min(uncomputed, budget,
  max_prefill_chunk_size)`` further cut to what the free pages can hold;
* then new requests are admitted from the head of the waiting queue, in order, never skipping
  the head, while a state slot is free and the pools stay above a watermark.

When pages run out: a decode makes room by preempting the *newest* running request, again and
again, possibly itself; the *oldest* running prefill may do the same to get a non-empty
portion, younger prefills wait; a newcomer never preempts anyone.  Preemption is recompute:
the victim's pages are returned, its computed count drops to zero, and it goes to the *front*
of the waiting queue, keeping the tokens it has generated; when it is admitted again its
prompt and generated tokens are prefilled anew (engine/scheduler.py:136-159).

With several cache groups a step needs the same number of new pages from every pool, so every
count below is taken from the fullest pool.
"""
from __future__ import annotations

import logging
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional

from ..cache.manager import CacheManager
from ..config.engine_config import SchedulerConfig
from .request import FinishReason, Request, RequestStatus

logger = logging.getLogger(__name__)


@dataclass
class SchedulerOutput:
    prefill_batch: List[Request] = field(default_factory=list)
    decode_batch: List[Request] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    num_batched_tokens: int = 0

    def is_empty(self) -> bool:
        return not self.prefill_batch and not self.decode_batch

    @property
    def scheduled(self) -> List[Request]:
        """Every request of the step, portions of prompts first, then single decoded tokens."""
        return self.prefill_batch + self.decode_batch


class Scheduler:
    def __init__(self, cache: CacheManager, config: Optional[SchedulerConfig] = None) -> None:
        self.cache = cache
        self.config = config or SchedulerConfig()
        self.config.max_model_len = min(self.config.max_model_len, cache.max_model_len)

        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.requests: Dict[str, Request] = {}

        self._watermark_pages = max(1, int(cache.num_total_pages * self.config.watermark))
        self.num_preemptions = 0
        self.num_finished = 0
        # Called with the request after it left the scheduler for good (finished or aborted).
        self.on_request_released: Optional[Callable[[Request], None]] = None

    # ------------------------------------------------------------------ queue
    def add_request(self, request: Request) -> None:
        limit = self.config.max_model_len
        if request.num_prompt_tokens >= limit:
            raise ValueError(
                f"prompt of {request.num_prompt_tokens} tokens does not fit in "
                f"max_model_len={limit} (at least one token must remain for generation)"
            )
        if request.num_prompt_tokens + request.sampling_params.max_tokens > limit:
            raise ValueError(
                f"prompt of {request.num_prompt_tokens} tokens plus "
                f"max_tokens={request.sampling_params.max_tokens} exceeds max_model_len={limit}"
            )
        if request.request_id in self.requests:
            raise ValueError(f"request id {request.request_id!r} is already in the scheduler")
        request.cache = self.cache.new_sequence(request.request_id)
        self.requests[request.request_id] = request
        self.waiting.append(request)

    def get_request(self, request_id: str) -> Optional[Request]:
        return self.requests.get(request_id)

    def abort_request(self, request_id: str) -> bool:
        request = self.requests.get(request_id)
        if request is None or request.finished:
            return False
        request.finish(FinishReason.ABORT)
        self._release(request)
        if request in self.waiting:
            self.waiting.remove(request)
        if request in self.running:
            self.running.remove(request)
        self.requests.pop(request_id, None)
        return True

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    @property
    def num_waiting(self) -> int:
        return len(self.waiting)

    @property
    def num_running(self) -> int:
        return len(self.running)

    # ------------------------------------------------------------------ release and preemption
    def _release(self, request: Request) -> None:
        self.cache.free(request.cache)
        self.cache.release_slot(request.cache)
        if self.on_request_released is not None:
            self.on_request_released(request)

    def _preempt(self, request: Request, output: SchedulerOutput) -> None:
        self.cache.reset_for_recompute(request.cache)
        self.cache.release_slot(request.cache)
        request.status = RequestStatus.PREEMPTED
        request.num_preemptions += 1
        self.num_preemptions += 1
        if request in self.running:
            self.running.remove(request)
        self.waiting.appendleft(request)
        output.preempted.append(request)
        logger.debug("preempted %s (%d so far)", request.request_id, self.num_preemptions)

    def _make_room(self, request: Request, num_tokens: int, output: SchedulerOutput) -> bool:
        """Preempt from the back of ``running`` until ``request`` can grow by ``num_tokens``.

        The victim is always the newest request, even when that is the caller: skipping past it
        to an older one is what would let a late arrival starve an early one.
        """
        while not self.cache.can_append(request.cache, num_tokens):
            if not self.running:
                return False
            victim = self.running[-1]
            self._preempt(victim, output)
            if victim is request:
                return False
        return True

    # ------------------------------------------------------------------ one step
    def schedule(self) -> SchedulerOutput:
        output = SchedulerOutput()
        self._reap_finished()
        budget = self.config.max_num_batched_tokens
        budget = self._schedule_decodes(output, budget)
        budget = self._schedule_running_prefills(output, budget)
        self._admit_waiting(output, budget)
        output.num_batched_tokens = len(output.decode_batch) + sum(
            request.current_chunk_size for request in output.prefill_batch
        )
        return output

    def _reap_finished(self) -> None:
        keep = []
        for request in self.running:
            if request.finished:
                self._release(request)
                self.requests.pop(request.request_id, None)
                self.num_finished += 1
            else:
                keep.append(request)
        self.running = keep

    def _schedule_decodes(self, output: SchedulerOutput, budget: int) -> int:
        for request in list(self.running):
            if request.status is not RequestStatus.RUNNING_DECODE or request not in self.running:
                continue
            if budget <= 0:
                break
            if not self._make_room(request, 1, output) or not self.cache.append_slots(
                request.cache, 1
            ):
                if request in self.running:
                    self._preempt(request, output)
                continue
            request.current_chunk_size = 1
            output.decode_batch.append(request)
            budget -= 1
        return budget

    def _largest_portion(self, request: Request, spare_pages: int) -> int:
        """Tokens that fit in the request's pages plus ``spare_pages`` new ones per pool."""
        cache = self.cache
        blocks = min(
            request.cache.num_logical_blocks + max(0, spare_pages), cache.max_blocks_per_seq
        )
        room = min(
            blocks * cache.page_size - request.num_computed_tokens,
            cache.max_model_len - request.num_computed_tokens,
        )
        return max(0, room)

    def _wanted_portion(self, request: Request, budget: int) -> int:
        return min(request.num_uncomputed_tokens, budget, self.config.max_prefill_chunk_size)

    def _schedule_running_prefills(self, output: SchedulerOutput, budget: int) -> int:
        oldest = True
        for request in list(self.running):
            if request.status is not RequestStatus.RUNNING_PREFILL or request not in self.running:
                continue
            if budget <= 0:
                break
            is_oldest, oldest = oldest, False

            wanted = self._wanted_portion(request, budget)
            portion = min(wanted, self._largest_portion(request, self.cache.num_free_pages()))
            while portion <= 0 and is_oldest and self.running and self.running[-1] is not request:
                self._preempt(self.running[-1], output)
                portion = min(wanted, self._largest_portion(request, self.cache.num_free_pages()))
            if portion <= 0 or not self.cache.append_slots(request.cache, portion):
                continue
            request.current_chunk_size = portion
            output.prefill_batch.append(request)
            budget -= portion
        return budget

    def _admit_waiting(self, output: SchedulerOutput, budget: int) -> None:
        while self.waiting and budget > 0 and len(self.running) < self.config.max_num_seqs:
            request = self.waiting[0]
            if not self.cache.acquire_slot(request.cache):
                break
            spare = self.cache.num_free_pages() - self._watermark_pages
            portion = min(self._wanted_portion(request, budget), self._largest_portion(request, spare))
            if portion <= 0 or not self.cache.append_slots(request.cache, portion):
                # Roll the admission back and stop: the head of the queue is never skipped.
                self.cache.reset_for_recompute(request.cache)
                self.cache.release_slot(request.cache)
                break
            self.waiting.popleft()
            request.status = RequestStatus.RUNNING_PREFILL
            request.current_chunk_size = portion
            self.running.append(request)
            output.prefill_batch.append(request)
            budget -= portion

    # ------------------------------------------------------------------ reporting
    def stats(self) -> Dict[str, float]:
        return {
            "num_running": float(len(self.running)),
            "num_waiting": float(len(self.waiting)),
            "num_preemptions": float(self.num_preemptions),
            "num_finished": float(self.num_finished),
            **self.cache.stats(),
        }
